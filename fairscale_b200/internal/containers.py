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


def _rebuild_ordered(x: "OrderedDict", walk: Callable) -> "OrderedDict":
    # subclasses of OrderedDict (model outputs of some libraries) carry attributes beside their items: both are kept
    out = type(x)()
    for key in x:
        out[key] = walk(x[key])
    vars(out).update(vars(x))
    return out


# (test, how to rebuild around the mapped children), tried from top to bottom: the order matters where one kind is a special
# case of another (OrderedDict before dict, PackedSequence and namedtuples before tuple)
_KINDS: List[Tuple[Callable[[Any], bool], Callable[[Any, Callable], Any]]] = [
    (lambda x: isinstance(x, OrderedDict), _rebuild_ordered),
    # a PackedSequence is an immutable named tuple: rebuild it around the mapped data (the reference calls fn for its side
    # effects only and returns the input, which loses casts and device moves)
    (lambda x: isinstance(x, PackedSequence), lambda x, walk: x._replace(data=walk(x.data))),
    (lambda x: isinstance(x, dict), lambda x, walk: {key: walk(x[key]) for key in x}),
    (_is_namedtuple, lambda x, walk: type(x)(*map(walk, x))),
    (lambda x: isinstance(x, list), lambda x, walk: list(map(walk, x))),
    (lambda x: isinstance(x, tuple), lambda x, walk: tuple(map(walk, x))),
    (lambda x: isinstance(x, set), lambda x, walk: set(map(walk, x))),
]


def apply_to_type(type_fn: Callable[[Any], bool], fn: Callable, container: Any) -> Any:
    """``container`` rebuilt with ``fn(leaf)`` in the place of every leaf that ``type_fn`` accepts.  Dicts, ordered dicts (and
    their subclasses, attributes included), lists, tuples, named tuples, sets and packed sequences are walked and come back
    as the same kind; every other object is a leaf and, unless ``type_fn`` accepts it, is returned untouched."""

    def walk(x: Any) -> Any:
        if type_fn(x):
            return fn(x)
        for is_kind, rebuild in _KINDS:
            if is_kind(x):
                return rebuild(x, walk)
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
