"""Flat parameter storage for a module tree.

API and state-dict parity with fairscale/nn/misc/flatten_params_wrapper.py:42-530:
``FlatParameter`` (views, metadata, pickling) and ``FlattenParamsWrapper`` (several flat
groups, shared parameters, ``unflatten_params`` context, ``flat_state_dict``, key
prefix ``_fpw_module.`` hidden from checkpoints).

Why it matters on B200: one contiguous, 16-byte aligned flat buffer per FSDP unit is
what the NVLink all-gather / reduce-scatter kernels and the multi-tensor Adam kernel
operate on — one collective and one optimizer launch per unit instead of one per
tensor — and views of it are valid TMA sources for the GEMM kernels.
"""

from __future__ import annotations

from contextlib import contextmanager
from itertools import chain
from typing import (
    TYPE_CHECKING,
    Any,
    Callable,
    Dict,
    Generator,
    Iterator,
    List,
    NamedTuple,
    Optional,
    Sequence,
    Set,
    Tuple,
    Union,
    cast,
)

import torch
from torch import Tensor, nn

from ...internal.state_dict import replace_by_prefix_

if TYPE_CHECKING:
    from collections import OrderedDict  # noqa: F401

# Switch read by FSDP's local-state-dict loading, which wants keys passed through untouched.
_enable_pre_load_state_dict_hook = True

# (module path, owning module, attribute name)
ParamInfo = Tuple[str, nn.Module, str]
# (module path, path of first owner, module, attr, first owner module, first owner attr)
SharedParamInfo = Tuple[str, str, nn.Module, str, nn.Module, str]


class FlatParameter(nn.Parameter):
    """A 1-D parameter made by concatenating other parameters.

    ``self.data`` may later be swapped for a shard of the full buffer; the recorded
    numels/shapes always describe the unsharded layout.
    """

    def __new__(cls, params: Sequence[Union[nn.Parameter, Tensor]], requires_grad: bool = True) -> "FlatParameter":
        if not isinstance(params, (list, tuple)) or len(params) == 0:
            raise ValueError("An non-empty list or tuple argument is needed")
        if not all(isinstance(p, (nn.Parameter, Tensor)) for p in params):
            raise ValueError("List items need to be Parameter types")
        if any(isinstance(p, FlatParameter) for p in params):
            raise ValueError("Nesting FlatParameter is not supported")
        pieces = [p.detach().reshape(-1) for p in params]
        flat = pieces[0].clone() if len(pieces) == 1 else torch.cat(pieces, 0)
        return super().__new__(cls, flat, requires_grad=requires_grad)  # type: ignore[call-arg]

    def __init__(self, params: Sequence[Union[nn.Parameter, Tensor]], requires_grad: bool = True):
        self._param_numels: List[int] = [p.numel() for p in params]
        self._param_shapes: List[torch.Size] = [p.size() for p in params]
        assert self.numel() <= sum(self._param_numels), (
            f"Something wrong with __new__ method, {self.numel()} vs. {sum(self._param_numels)}"
        )
        # filled in by FlattenParamsWrapper
        self._param_infos: List[ParamInfo] = []
        self._shared_param_infos: List[SharedParamInfo] = []

    @property
    def full_numel(self) -> int:
        return sum(self._param_numels)

    def get_param_views(self, external_data: Optional[Tensor] = None) -> Iterator[Tensor]:
        """Views with the original shapes into ``self`` (or into ``external_data``)."""
        total = self.full_numel
        assert self.data.numel() <= total, f"Incorrect internal state {self.data.numel()} vs. {total}"
        src = self if external_data is None else external_data
        if src.numel() != total:
            raise ValueError(f"Incorrect numel of supplied data: got {src.numel()} but expected {total}")
        return (piece.view(shape) for piece, shape in zip(src.split(self._param_numels), self._param_shapes))

    def get_param_views_for_forward(self) -> Iterator[Tensor]:
        """Views for the wrapped module's forward.  When a gradient will be needed they come from
        :class:`_FlatViews` and carry their :class:`GradArena` window, so weight gradients can be written
        straight into the flat gradient."""
        if not (self.requires_grad and torch.is_grad_enabled()) or self.data.numel() != self.full_numel:
            return self.get_param_views()
        arena = getattr(self, "_grad_arena", None)
        if arena is None or arena.total != self.full_numel:
            arena = self._grad_arena = GradArena(self.full_numel)
        views = _FlatViews.apply(self, self._param_numels, self._param_shapes, arena)
        off = 0
        for v, n, shp in zip(views, self._param_numels, self._param_shapes):
            v._fsb_grad_slot = (arena, off, shp)
            off += n
        return iter(views)

    def metadata(self) -> Tuple[List[str], List[torch.Size], List[int]]:
        """``(names, shapes, numels)`` of the original parameters, names relative to the wrapped module."""
        names = [f"{path}.{attr}" if path else attr for path, _, attr in self._param_infos]
        return names, self._param_shapes, self._param_numels

    # -- pickling: the tensor travels as data, the bookkeeping as state
    def __setstate__(self, state: Tuple[Any, Any, Any, Any]) -> None:
        self._param_numels, self._param_shapes, self._param_infos, self._shared_param_infos = state
        assert self.numel() <= sum(self._param_numels), (
            f"Incorrect pickling {self.numel()} vs. {sum(self._param_numels)}"
        )

    def __reduce_ex__(self, proto: int) -> Tuple[Any, Any, Any]:
        return (
            FlatParameter,
            ([self.data], self.requires_grad),
            (self._param_numels, self._param_shapes, self._param_infos, self._shared_param_infos),
        )


# Optional source of gradient buffers: ``fn(numel, dtype, device) -> Tensor | None``.  The data-parallel wrapper points it
# at the symmetric heap of its NVLink workspace, so that weight-gradient GEMMs write where the peers' reduce-scatter
# kernels read and no staging copy is needed; None (the default) or a None result means ordinary device memory.
_GRAD_BUFFER_PROVIDER: Optional[Callable[[int, torch.dtype, torch.device], Optional[Tensor]]] = None


def set_grad_buffer_provider(fn: Optional[Callable[[int, torch.dtype, torch.device], Optional[Tensor]]]) -> None:
    global _GRAD_BUFFER_PROVIDER
    _GRAD_BUFFER_PROVIDER = fn


def _new_grad_buffer(total: int, dtype: torch.dtype, device: torch.device) -> Tensor:
    if _GRAD_BUFFER_PROVIDER is not None:
        buf = _GRAD_BUFFER_PROVIDER(total, dtype, device)
        if buf is not None:
            return buf
    return torch.empty(total, dtype=dtype, device=device)


class GradArena:
    """Per-flat-parameter landing zone for weight gradients.

    Views handed to the wrapped module carry ``_fsb_grad_slot = (arena, offset, shape)``.  A kernel that
    produces the gradient of such a view (e.g. the wgrad GEMM) asks :meth:`slot` for the matching window of
    one flat buffer and writes there directly; when autograd later assembles the flat parameter's gradient,
    windows that were filled in place need no copy, which removes the ``torch.cat`` of all per-parameter
    gradients (one full read+write of the gradient per unit per step).
    """

    def __init__(self, total: int):
        self.total = total
        self.buffer: Optional[Tensor] = None
        self.claimed: Set[int] = set()

    def slot(self, offset: int, shape: torch.Size, dtype: torch.dtype, device: torch.device) -> Optional[Tensor]:
        """Window for the gradient of the view at ``offset`` — at most once per backward (a second use of the
        same weight must go through autograd's own accumulation)."""
        if offset in self.claimed:
            return None
        if self.buffer is None:
            self.buffer = _new_grad_buffer(self.total, dtype, device)
        elif self.buffer.dtype != dtype or self.buffer.device != device:
            return None
        self.claimed.add(offset)
        return self.buffer[offset : offset + shape.numel()].view(shape)

    def take(self, dtype: torch.dtype, device: torch.device) -> Tensor:
        buf = self.buffer
        if buf is None or buf.dtype != dtype or buf.device != device:
            buf = _new_grad_buffer(self.total, dtype, device)
        self.buffer = None
        self.claimed = set()
        return buf


def grad_slot_for(weight: Tensor) -> Optional[Tensor]:
    """The in-place gradient window of ``weight`` if it is a view handed out by a flat parameter, else None."""
    info = getattr(weight, "_fsb_grad_slot", None)
    if info is None:
        return None
    arena, offset, shape = info
    return arena.slot(offset, shape, weight.dtype, weight.device)


class _FlatViews(torch.autograd.Function):
    """flat parameter -> per-parameter views; backward gathers the views' gradients into one flat buffer,
    skipping those already written in place through the :class:`GradArena`."""

    @staticmethod
    def forward(ctx: Any, flat: Tensor, numels: List[int], shapes: List[torch.Size], arena: GradArena):  # type: ignore[override]
        ctx.numels, ctx.shapes, ctx.arena = numels, shapes, arena
        ctx.flat_meta = (flat.dtype, flat.device)
        return tuple(t.view(s) for t, s in zip(flat.split(numels), shapes))

    @staticmethod
    def backward(ctx: Any, *grads: Any):  # type: ignore[override]
        dtype, device = ctx.flat_meta
        claimed = set(ctx.arena.claimed)
        buf = ctx.arena.take(dtype, device)
        off = 0
        for g, n in zip(grads, ctx.numels):
            window = buf[off : off + n]
            if g is None:
                window.zero_()
            elif off in claimed and g.data_ptr() == window.data_ptr() and g.dtype == dtype:
                pass  # produced in place
            else:
                window.copy_(g.reshape(-1))
            off += n
        return buf, None, None, None


ParamGroups = Optional[Union[List[List[nn.Parameter]], List[nn.Parameter]]]


class FlattenParamsWrapper(nn.Module):
    """Replace (groups of) a module's parameters by flat parameters ``flat_param_<name>``.

    Args:
        module: module to wrap.
        param_list: parameters to flatten — a list (one group) or a list of lists (one
            flat parameter per inner list).  ``None`` flattens all parameters.  A
            parameter may not appear in two groups; shared parameters inside one
            group are stored once.
        flat_param_names: suffixes for the registered names (default ``"0", "1", …``).
    """

    def __init__(self, module: nn.Module, param_list: ParamGroups = None, flat_param_names: Optional[List[str]] = None):
        super().__init__()
        self._fpw_module = module
        self.is_flattened = False

        if param_list is None:
            param_list = list(module.parameters())
        if len(param_list) > 0 and isinstance(param_list[0], nn.Parameter):
            param_list = [cast(List[nn.Parameter], param_list)]

        # (module, attr) pairs survive parameter objects being replaced
        self.num_params_managed = 0
        self._param_sets: List[Set[Tuple[nn.Module, str]]] = []
        seen: Set[nn.Parameter] = set()
        for group in cast(List[List[nn.Parameter]], param_list):
            unique = set(group)
            self.num_params_managed += len(unique)
            seen |= unique
            owners = {
                (m, n) for m in self.modules() for n, p in m.named_parameters(recurse=False) if p in unique
            }
            if owners:
                self._param_sets.append(owners)
        if len(seen) != self.num_params_managed:
            raise ValueError(f"Incorrect param groups {len(seen)} vs {self.num_params_managed}")

        if flat_param_names is None:
            flat_param_names = [str(i) for i in range(len(self._param_sets))]
        if len(flat_param_names) != len(self._param_sets):
            raise ValueError("Names and number of param lists must be equal")
        if len(set(flat_param_names)) != len(flat_param_names):
            raise ValueError("Each flat param must be given a unique name")
        self.flat_param_names = [f"flat_param_{n}" for n in flat_param_names]

        self.flat_params: List[nn.Parameter] = []
        for owners in self._param_sets:
            params, infos, shared_infos = self._init_flatten_params(owners)
            fp = FlatParameter(params, params[0].requires_grad)
            fp._param_infos = infos
            fp._shared_param_infos = shared_infos
            self.flat_params.append(fp)
        self._flatten_params(self.flat_params)

        self._register_state_dict_hook(_post_state_dict_hook)
        self._register_load_state_dict_pre_hook(_pre_load_state_dict_hook)
        self._auto_unflatten_state_dict = True

    # ------------------------------------------------------------------ accessors
    @property
    def module(self) -> Any:
        return self._fpw_module

    @property
    def flat_param(self) -> nn.Parameter:
        assert len(self.flat_params) == 1, (
            f"Incorrect access to flat_param: len(self.flat_params)={len(self.flat_params)}"
        )
        return self.flat_params[0]

    @property
    def _param_infos(self) -> Iterator[ParamInfo]:
        return chain.from_iterable(p._param_infos for p in self.flat_params)  # type: ignore[attr-defined]

    @property
    def _shared_param_infos(self) -> Iterator[SharedParamInfo]:
        return chain.from_iterable(p._shared_param_infos for p in self.flat_params)  # type: ignore[attr-defined]

    # ------------------------------------------------------------------ flatten / unflatten
    def _init_flatten_params(
        self, owners: Set[Tuple[nn.Module, str]]
    ) -> Tuple[List[nn.Parameter], List[ParamInfo], List[SharedParamInfo]]:
        """Collect, in module-traversal order, the distinct parameters of one group."""
        first_owner: Dict[nn.Parameter, ParamInfo] = {}
        infos: List[ParamInfo] = []
        shared: List[SharedParamInfo] = []
        params: List[nn.Parameter] = []
        by_dtype: Dict[torch.dtype, List[str]] = {}
        for path, mod in self.named_modules():
            for attr, p in mod.named_parameters(recurse=False):
                by_dtype.setdefault(p.dtype, []).append(path)
                if (mod, attr) not in owners:
                    continue
                if p in first_owner:
                    o_path, o_mod, o_attr = first_owner[p]
                    shared.append((path, o_path, mod, attr, o_mod, o_attr))
                else:
                    first_owner[p] = (path, mod, attr)
                    infos.append((path, mod, attr))
                    params.append(p)
        if len({p.dtype for p in params}) != 1:
            detail = " \n ".join(f"{dt}: {','.join(v)}" for dt, v in by_dtype.items())
            raise AssertionError(f"expects all parameters to have same dtype: {detail}")
        assert len({p.requires_grad for p in params}) == 1, (
            f"expects all parameters to have same requires_grad {owners}"
        )
        assert len(params) == len(set(params)), "params list should not have dups"
        return params, infos, shared

    def _flatten_params(self, flat_params: List[nn.Parameter]) -> None:
        assert not self.is_flattened
        self.is_flattened = True
        assert len(self.flat_param_names) == len(flat_params), f"{len(self.flat_param_names)} vs. {len(flat_params)}"
        for name, fp in zip(self.flat_param_names, flat_params):
            self.register_parameter(name, fp)
        self.flat_params = flat_params
        for _, mod, attr in self._param_infos:
            delattr(mod, attr)
        for _, _, mod, attr, _, _ in self._shared_param_infos:
            delattr(mod, attr)
        self._unflatten_params_as_views()

    def _unflatten_params(self, external_data: Optional[List[Optional[Tensor]]] = None) -> None:
        """Turn the wrapped module back into one with ordinary parameters."""
        assert self.is_flattened or external_data is not None
        self.is_flattened = False
        views = self.get_param_views(external_data)
        for (_, mod, attr), v in zip(self._param_infos, views):
            if hasattr(mod, attr):
                delattr(mod, attr)
            mod.register_parameter(attr, nn.Parameter(v))
        for _, _, mod, attr, o_mod, o_attr in self._shared_param_infos:
            if hasattr(mod, attr):
                delattr(mod, attr)
            mod.register_parameter(attr, getattr(o_mod, o_attr))
        if hasattr(self._fpw_module, "_unflattened_param_views"):
            delattr(self._fpw_module, "_unflattened_param_views")
        for name in self.flat_param_names:
            delattr(self, name)
        self.flat_params = []

    def _unflatten_params_as_views(self) -> None:
        """(Re)point the original attribute names at views of the current flat data."""
        assert self.is_flattened
        views: List[Tensor] = []
        fwd_views = chain.from_iterable(p.get_param_views_for_forward() for p in self.flat_params)  # type: ignore[attr-defined]
        for (_, mod, attr), v in zip(self._param_infos, fwd_views):
            setattr(mod, attr, v)  # plain attribute: the view is not an nn.Parameter
            views.append(v)
        # checkpoint_wrapper consults this to decide whether outputs need grad
        setattr(self._fpw_module, "_unflattened_param_views", views)
        for _, _, mod, attr, o_mod, o_attr in self._shared_param_infos:
            setattr(mod, attr, getattr(o_mod, o_attr))

    @contextmanager
    def unflatten_params(self, flat_params: Optional[List[Tensor]] = None) -> Generator:
        """Temporarily expose ordinary parameters (optionally backed by ``flat_params``)."""
        assert flat_params is None or self.is_flattened, (
            "Unflattening with external flat_param requires current instance to be flattened"
        )
        was_flat = self.is_flattened
        if was_flat:
            saved = self.flat_params
            self._unflatten_params(cast(Optional[List[Optional[Tensor]]], flat_params))
        try:
            yield
        finally:
            if was_flat:
                self._flatten_params(saved)

    # ------------------------------------------------------------------ module plumbing
    def __getattr__(self, name: str) -> Any:
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)

    def __getitem__(self, key: int) -> Any:
        return self.module.__getitem__(key)

    def state_dict(self, *args: Any, **kwargs: Any) -> Any:
        """Unflattened state dict of the wrapped module (flat inside ``flat_state_dict``)."""
        if self.is_flattened and self._auto_unflatten_state_dict:
            with self.unflatten_params():
                return super().state_dict(*args, **kwargs)
        return super().state_dict(*args, **kwargs)

    def flat_state_dict(self, *args: Any, **kwargs: Any) -> Dict[str, Any]:
        assert self.is_flattened
        with self._no_auto_unflatten_state_dict():
            return self.state_dict(*args, **kwargs)

    @contextmanager
    def _no_auto_unflatten_state_dict(self) -> Generator:
        prev = self._auto_unflatten_state_dict
        self._auto_unflatten_state_dict = False
        try:
            yield
        finally:
            self._auto_unflatten_state_dict = prev

    def load_state_dict(  # type: ignore[override]
        self, state_dict: Union[Dict[str, Tensor], "OrderedDict[str, Tensor]"], strict: bool = True
    ) -> NamedTuple:
        """Accept either a flat (``flat_param_*`` keys) or an unflattened state dict."""
        has_flat_keys = any(k.startswith("flat_param_") for k in state_dict.keys())
        if self.num_params_managed > 0 and self.is_flattened and not has_flat_keys:
            with self.unflatten_params():
                return super().load_state_dict(state_dict, strict)
        if "flat_param" in state_dict:  # key used before multiple groups existed
            state_dict["flat_param_0"] = state_dict.pop("flat_param")
        return super().load_state_dict(state_dict, strict)

    def forward(self, *inputs: Any, **kwinputs: Any) -> Any:
        self._unflatten_params_as_views()
        return self.module(*inputs, **kwinputs)

    def get_param_views(self, external_data_list: Optional[List[Optional[Tensor]]] = None) -> Iterator[Tensor]:
        params = self.flat_params
        if external_data_list is None:
            external_data_list = [None] * len(params)
        assert len(external_data_list) == len(params), (
            f"Incorrect external data list: {len(external_data_list)} vs. {len(params)}"
        )
        return chain.from_iterable(
            p.get_param_views(d) for p, d in zip(params, external_data_list)  # type: ignore[attr-defined]
        )

    def metadata(self, flat_param_idx: int) -> Tuple[List[str], Sequence[torch.Size], List[int]]:
        return self.flat_params[flat_param_idx].metadata()  # type: ignore[attr-defined]


def _post_state_dict_hook(
    module: nn.Module, state_dict: "OrderedDict[str, Tensor]", prefix: str, *args: Any
) -> "OrderedDict[str, Tensor]":
    replace_by_prefix_(state_dict, prefix + "_fpw_module.", prefix)
    return state_dict


def _pre_load_state_dict_hook(
    state_dict: Union[Dict[str, Tensor], "OrderedDict[str, Tensor]"], prefix: str, *args: Any
) -> None:
    if not _enable_pre_load_state_dict_hook:
        return
    inner = prefix + "_fpw_module."
    replace_by_prefix_(state_dict, prefix, inner)
    # flat parameters are registered on the wrapper itself, one level above the wrapped module
    for key in list(state_dict.keys()):
        if key.startswith(inner + "flat_param"):
            leaf = key.rsplit(".", 1)[-1]
            assert leaf.startswith("flat_param_"), leaf
            replace_by_prefix_(state_dict, key, prefix + leaf)
