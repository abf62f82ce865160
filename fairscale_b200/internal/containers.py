"""Recursive helpers over nested python containers that hold tensors.

Behavioural parity with fairscale/internal/containers.py:16-158 (apply_to_tensors,
pack_kwargs/unpack_kwargs, split_non_tensors/unpack_non_tensors).  The traversal is
written as a single dispatcher keyed on the container kind so that namedtuples,
OrderedDicts, sets and PackedSequence keep their concrete type.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
from torch.nn.utils.rnn import PackedSequence


def _is_namedtuple(x: Any) -> bool:
    return isinstance(x, tuple) and hasattr(x, "_fields") and hasattr(x, "_make")


def apply_to_type(type_fn: Callable[[Any], bool], fn: Callable, container: Any) -> Any:
    """Map ``fn`` over every leaf for which ``type_fn(leaf)`` is true.

    Containers are rebuilt with the same concrete type; other leaves are returned
    unchanged.  Dict values are mutated through ``__dict__`` for objects that are
    themselves dict-like holders (``OrderedDict`` subclasses keep extra attributes).
    """

    def walk(x: Any) -> Any:
        if type_fn(x):
            return fn(x)
        if isinstance(x, OrderedDict):
            out = x.__class__()
            for k, v in x.items():
                out[k] = walk(v)
            out.__dict__.update(x.__dict__)
            return out
        if isinstance(x, PackedSequence):
            # a PackedSequence is an immutable named tuple: rebuild it around the mapped data (the reference calls fn for
            # its side effects only and returns the input, which loses casts and device moves)
            return x._replace(data=walk(x.data))
        if isinstance(x, dict):
            return {k: walk(v) for k, v in x.items()}
        if _is_namedtuple(x):
            return type(x)(*(walk(v) for v in x))
        if isinstance(x, list):
            return [walk(v) for v in x]
        if isinstance(x, tuple):
            return tuple(walk(v) for v in x)
        if isinstance(x, set):
            return {walk(v) for v in x}
        return x

    return walk(container)


def apply_to_tensors(fn: Callable, container: Any) -> Any:
    """Recursively apply ``fn`` to every ``torch.Tensor`` in ``container``."""
    return apply_to_type(torch.is_tensor, fn, container)


def to_np(tensor_or_container: Any) -> Any:
    """Convert all tensors in a container to numpy arrays (CPU)."""
    return apply_to_type(torch.is_tensor, lambda t: t.detach().cpu().numpy(), tensor_or_container)


def from_np(ndarray_or_container: Any) -> Any:
    """Convert all numpy arrays in a container to tensors."""
    return apply_to_type(lambda x: isinstance(x, np.ndarray), torch.from_numpy, ndarray_or_container)


def pack_kwargs(*args: Any, **kwargs: Any) -> Tuple[Tuple[str, ...], Tuple[Any, ...]]:
    """Turn ``(*args, **kwargs)`` into ``(kwarg_keys, flat_args)``.

    ``autograd.Function.apply`` only takes positional arguments; the keyword
    values are appended after the positionals and their names returned separately.
    """
    keys = tuple(kwargs.keys())
    flat = tuple(args) + tuple(kwargs[k] for k in keys)
    return keys, flat


def unpack_kwargs(kwarg_keys: Sequence[str], flat_args: Sequence[Any]) -> Tuple[Tuple[Any, ...], Dict[str, Any]]:
    """Inverse of :func:`pack_kwargs`."""
    n_kw = len(kwarg_keys)
    assert n_kw <= len(flat_args), f"too many keys {n_kw} vs. {len(flat_args)}"
    if n_kw == 0:
        return tuple(flat_args), {}
    n_pos = len(flat_args) - n_kw
    return tuple(flat_args[:n_pos]), dict(zip(kwarg_keys, flat_args[n_pos:]))


def split_non_tensors(
    mixed: Union[torch.Tensor, Tuple[Any, ...]]
) -> Tuple[Tuple[torch.Tensor, ...], Optional[Dict[str, List[Any]]]]:
    """Separate tensors from everything else in a flat tuple.

    Returns ``(tensors, packed)`` where ``packed`` is ``None`` for a bare tensor,
    otherwise ``{"is_tensor": [...], "objects": [...]}`` which
    :func:`unpack_non_tensors` uses to restore the original order.
    """
    if isinstance(mixed, torch.Tensor):
        return (mixed,), None
    tensors: List[torch.Tensor] = []
    packed: Dict[str, List[Any]] = {"is_tensor": [], "objects": []}
    for item in mixed:
        flag = isinstance(item, torch.Tensor)
        packed["is_tensor"].append(flag)
        (tensors if flag else packed["objects"]).append(item)
    return tuple(tensors), packed


def unpack_non_tensors(
    tensors: Tuple[torch.Tensor, ...], packed_non_tensors: Optional[Dict[str, List[Any]]]
) -> Tuple[Any, ...]:
    """Inverse of :func:`split_non_tensors`."""
    if packed_non_tensors is None:
        return tensors
    assert isinstance(packed_non_tensors, dict), type(packed_non_tensors)
    flags = packed_non_tensors["is_tensor"]
    objects = packed_non_tensors["objects"]
    assert len(tensors) + len(objects) == len(flags), (
        f"len(tensors) {len(tensors)} len(objects) {len(objects)} len(is_tensor) {len(flags)}"
    )
    t_iter, o_iter = iter(tensors), iter(objects)
    return tuple(next(t_iter) if f else next(o_iter) for f in flags)
