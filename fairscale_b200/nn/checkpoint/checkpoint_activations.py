"""Activation checkpointing as a module wrapper.

Parity: fairscale/nn/checkpoint/checkpoint_activations.py:25-353 — ``checkpoint_wrapper``
keeps only a block's inputs in forward and recomputes the block in backward; it accepts
keyword arguments and non-tensor outputs, restores RNG and autocast state for the
recomputation, and can park the saved inputs in host memory.

Host offload uses pinned staging buffers and a dedicated copy stream with events, so the
device→host copy of one block's input overlaps the next block's compute, and the
host→device copy is issued ahead of the recomputation.
"""

from __future__ import annotations

import threading
import weakref
from contextlib import contextmanager, nullcontext
from typing import Any, Dict, Generator, List, Optional, Tuple

import torch
import torch.utils.checkpoint as torch_checkpoint
from torch import Tensor, nn

from ...internal.containers import pack_kwargs, split_non_tensors, unpack_kwargs, unpack_non_tensors
from .checkpoint_utils import patch_batchnorm


class _Flags(threading.local):
    def __init__(self) -> None:
        self.is_checkpointing = False
        self.is_recomputing = False
        self.is_checkpointing_disabled = False
        self.region_owners: List[Any] = []
        self.invocations: List[Dict[str, Any]] = []  # one scratch dict per checkpointed call that is running, innermost last


thread_local = _Flags()


@contextmanager
def _running_invocation(scratch: Dict[str, Any], mode: str) -> Generator[None, None, None]:
    scratch["_mode"] = mode  # "first": the no-grad forward; "replay": its repetition in backward
    thread_local.invocations.append(scratch)
    try:
        yield
    finally:
        thread_local.invocations.pop()


def checkpoint_invocations() -> List[Dict[str, Any]]:
    """Scratch dicts of the checkpointed calls that are running in this thread, innermost last.  One dict belongs to one call
    of a checkpointed module: it is current during the call's forward (``scratch["_mode"] == "first"``) and again during the
    repetition of exactly that call in backward (``"replay"``), whatever the order in which autograd gets to the calls of a
    step.  Layers with side effects keep what the repetition has to reuse there (e.g. SyncBatchNorm its batch statistics)."""
    return thread_local.invocations


@contextmanager
def _flag(name: str, value: bool = True) -> Generator[None, None, None]:
    prev = getattr(thread_local, name)
    setattr(thread_local, name, value)
    try:
        yield
    finally:
        setattr(thread_local, name, prev)


@contextmanager
def owning_checkpointed_regions(owner: Any) -> Generator[None, None, None]:
    """While this context is active, every checkpointed region that starts a forward is counted in
    ``owner._ckpt_outstanding`` until its backward (recomputation included) has run.  A parameter-sharding wrapper uses the
    count to keep its full parameters until the last region that will recompute with them is done."""
    thread_local.region_owners.append(owner)
    try:
        yield
    finally:
        thread_local.region_owners.pop()


def disable_checkpointing() -> Any:
    """Context in which wrapped modules run as if they were not checkpointed."""
    return _flag("is_checkpointing_disabled")


def enable_checkpointing() -> Any:
    return _flag("is_checkpointing")


def enable_recomputing() -> Any:
    return _flag("is_recomputing")


def is_checkpointing() -> bool:
    """True inside the first (no-grad) forward of a checkpointed module."""
    return thread_local.is_checkpointing


def is_recomputing() -> bool:
    """True inside the backward-time recomputation; use it to avoid repeating side effects."""
    return thread_local.is_recomputing


def checkpoint_wrapper(module: nn.Module, offload_to_cpu: bool = False) -> nn.Module:
    """Make every later call of ``module`` activation-checkpointed; returns the same object.

    Inner activations are dropped and recomputed; with ``offload_to_cpu`` the saved
    inputs (the "outer" activations) additionally live in pinned host memory between
    forward and backward.  No-op under ``torch.no_grad()`` and inside
    :func:`disable_checkpointing`.
    """
    patch_batchnorm(module)
    module._fsb_checkpointed = True  # type: ignore[assignment]  # wrappers may rely on the forward being replayed in backward
    module.forward = _CheckpointedForward(type(module).forward, module, offload_to_cpu)  # type: ignore[method-assign]
    return module


class _CheckpointedForward:
    """The ``forward`` of a wrapped module.  It reaches its module through a weak reference (a strong one would form a
    module <-> forward cycle that keeps the module alive until the garbage collector runs), and a deep copy of the
    module gets a forward that points at the copy, not at the original."""

    def __init__(self, original_forward: Any, module: nn.Module, offload_to_cpu: bool) -> None:
        self.original_forward = original_forward
        self.weak_self = weakref.ref(module)
        self.offload_to_cpu = offload_to_cpu

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        return _checkpointed_forward(self.original_forward, self.weak_self, self.offload_to_cpu, *args, **kwargs)

    def __deepcopy__(self, memo: Dict[int, Any]) -> "_CheckpointedForward":
        original = self.weak_self()
        owner = memo.get(id(original)) if original is not None else None  # the copy under construction, if we are part of one
        return _CheckpointedForward(self.original_forward, owner if owner is not None else original, self.offload_to_cpu)


def _checkpointed_forward(original_forward: Any, weak_self: Any, offload_to_cpu: bool, *args: Any, **kwargs: Any) -> Any:
    module = weak_self()
    if not torch.is_grad_enabled() or thread_local.is_checkpointing_disabled:
        return original_forward(module, *args, **kwargs)

    kwarg_keys, flat_args = pack_kwargs(module, *args, **kwargs)
    shared: Dict[str, Any] = {"offload": offload_to_cpu}
    # the dummy input guarantees the Function node is part of the graph even if no input needs grad
    out = CheckpointFunction.apply(torch.tensor([], requires_grad=True), original_forward, shared, kwarg_keys, *flat_args)
    needs_grad = shared["output_requires_grad"]
    if isinstance(out, torch.Tensor):
        return out if needs_grad else out.detach()
    out = [t if needs_grad else t.detach() for t in out]
    packed = shared["packed_non_tensor_outputs"]
    return unpack_non_tensors(tuple(out), packed) if packed else out


def get_rng_state() -> Dict[str, Any]:
    state = {"torch_rng_state": torch.get_rng_state()}
    if torch.cuda.is_available():
        state["cuda_rng_state"] = torch.cuda.get_rng_state()
    return state


def set_rng_state(state: Dict[str, Any]) -> None:
    torch.set_rng_state(state["torch_rng_state"])
    if torch.cuda.is_available():
        torch.cuda.set_rng_state(state["cuda_rng_state"])


def _autocast_snapshot() -> Optional[Dict[str, Any]]:
    if torch.is_autocast_enabled("cuda"):
        return {"device_type": "cuda", "dtype": torch.get_autocast_dtype("cuda")}
    if torch.is_autocast_enabled("cpu"):
        return {"device_type": "cpu", "dtype": torch.get_autocast_dtype("cpu")}
    return None


class _HostParking:
    """Device→pinned-host and back, on a side stream ordered by events."""

    _streams: Dict[int, Any] = {}

    @classmethod
    def _stream(cls, device: torch.device) -> Any:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in cls._streams:
            cls._streams[idx] = torch.cuda.Stream(device=idx)
        return cls._streams[idx]

    @classmethod
    def park(cls, t: Tensor) -> Tuple[Tensor, Any]:
        if not t.is_cuda:
            return t.to("cpu"), None
        side = cls._stream(t.device)
        side.wait_stream(torch.cuda.current_stream(t.device))
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        with torch.cuda.stream(side):
            host.copy_(t, non_blocking=True)
            done = torch.cuda.Event()
            done.record(side)
        t.record_stream(side)
        return host, done

    @classmethod
    def fetch(cls, host: Tensor, done: Any, device: torch.device) -> Tensor:
        if device.type != "cuda":
            return host.to(device)
        side = cls._stream(device)
        if done is not None:
            side.wait_event(done)
        with torch.cuda.stream(side):
            dev = host.to(device, non_blocking=True)
        torch.cuda.current_stream(device).wait_stream(side)
        dev.record_stream(torch.cuda.current_stream(device))
        return dev


def is_autocast_enabled() -> bool:
    """``torch.is_autocast_enabled()`` (the reference wraps it for very old torch versions)."""
    return torch.is_autocast_enabled()


@contextmanager
def autocast(enabled: bool) -> Generator:
    """CUDA autocast when ``enabled``, nothing otherwise (used to replay the forward's autocast state in recomputation)."""
    if enabled:
        with torch.autocast("cuda", enabled=True):
            yield
    else:
        yield


def _has_trainable_weights(module: nn.Module) -> bool:
    """True if ``module`` or a sub-module holds a weight that requires grad: an ``nn.Parameter``, or - under a flattening
    wrapper, which replaces parameters by plain tensor attributes that are views of its flat parameter - such a view.  The
    wrapper records its views on the module it wraps (``_unflattened_param_views``); a checkpointed sub-module of that module
    only sees them as attributes, so those are looked at as well."""
    if any(p.requires_grad for p in module.parameters()):
        return True
    if any(v.requires_grad for v in getattr(module, "_unflattened_param_views", [])):
        return True
    for m in module.modules():
        for v in vars(m).values():
            if isinstance(v, torch.Tensor) and v.requires_grad:
                return True
    return False


class CheckpointFunction(torch.autograd.Function):
    """Autograd node that runs ``run_function`` without grad and replays it in backward.

    Non-tensor outputs travel through ``parent_ctx_dict`` (autograd Functions can only
    return tensors); the caller merges them back.
    """

    @staticmethod
    def forward(  # type: ignore[override]
        ctx: Any,
        dummy_tensor_requires_grad: Tensor,
        run_function: Any,
        parent_ctx_dict: Dict[str, Any],
        kwarg_keys: Tuple[str, ...],
        *args: Any,
    ) -> Any:
        torch_checkpoint.check_backward_validity(args)
        ctx.region_owner = thread_local.region_owners[-1] if thread_local.region_owners else None
        if ctx.region_owner is not None:
            ctx.region_owner._ckpt_outstanding = getattr(ctx.region_owner, "_ckpt_outstanding", 0) + 1
        ctx.run_function = run_function
        ctx.kwarg_keys = kwarg_keys
        ctx.fwd_rng_state = get_rng_state()
        ctx.autocast = _autocast_snapshot()

        tensor_inputs, packed_inputs = split_non_tensors(args)
        if parent_ctx_dict["offload"]:
            ctx.fwd_device = tuple(t.device for t in tensor_inputs)
            ctx.grad_requirements = tuple(t.requires_grad for t in tensor_inputs)
            parked = [_HostParking.park(t) for t in tensor_inputs]
            ctx.park_events = [ev for _, ev in parked]
            tensor_inputs = tuple(h for h, _ in parked)
        else:
            ctx.fwd_device, ctx.grad_requirements, ctx.park_events = None, None, None
        ctx.save_for_backward(*tensor_inputs)
        ctx.packed_non_tensor_inputs = packed_inputs
        ctx.scratch = {}

        with torch.no_grad(), enable_checkpointing(), _running_invocation(ctx.scratch, "first"):
            f_args, f_kwargs = unpack_kwargs(kwarg_keys, args)
            outputs = run_function(*f_args, **f_kwargs)
            the_module = f_args[0]

        grad_src = ctx.grad_requirements if ctx.grad_requirements is not None else [t.requires_grad for t in tensor_inputs]
        parent_ctx_dict["output_requires_grad"] = _has_trainable_weights(the_module) or any(grad_src)

        if not isinstance(outputs, torch.Tensor):
            outputs, packed_outputs = split_non_tensors(outputs)
            parent_ctx_dict["packed_non_tensor_outputs"] = packed_outputs
        return outputs

    @staticmethod
    def backward(ctx: Any, *grads: Any) -> Tuple[Optional[Tensor], ...]:
        if not torch.autograd._is_checkpoint_valid():
            raise RuntimeError("Checkpointing is not compatible with .grad(), please use .backward() if possible")
        try:
            return CheckpointFunction._replay(ctx, *grads)
        finally:
            owner = ctx.region_owner
            if owner is not None and getattr(owner, "_ckpt_outstanding", 0) > 0:
                owner._ckpt_outstanding -= 1

    @staticmethod
    def _replay(ctx: Any, *grads: Any) -> Tuple[Optional[Tensor], ...]:
        saved: Tuple[Tensor, ...] = ctx.saved_tensors
        if ctx.fwd_device is not None:
            restored = []
            for t, dev, ev, need in zip(saved, ctx.fwd_device, ctx.park_events, ctx.grad_requirements):
                d = _HostParking.fetch(t, ev, dev).detach()
                d.requires_grad = need
                restored.append(d)
            tensor_inputs: Tuple[Tensor, ...] = tuple(restored)
        else:
            tensor_inputs = torch_checkpoint.detach_variable(saved)
        inputs = unpack_non_tensors(tensor_inputs, ctx.packed_non_tensor_inputs)

        # replay under the forward's RNG state so dropout masks match, then put the current state back
        rng_now = get_rng_state()
        set_rng_state(ctx.fwd_rng_state)
        amp = torch.autocast(**ctx.autocast) if ctx.autocast is not None else nullcontext()
        with torch.enable_grad(), enable_recomputing(), amp, _running_invocation(ctx.scratch, "replay"):
            f_args, f_kwargs = unpack_kwargs(ctx.kwarg_keys, inputs)
            outputs = ctx.run_function(*f_args, **f_kwargs)
            tensor_outputs, _ = split_non_tensors(outputs)
        set_rng_state(rng_now)

        live = [(o, g) for o, g in zip(tensor_outputs, grads) if o.requires_grad]
        if not live:
            raise RuntimeError("None of the outputs have requires_grad=True, this checkpoint() is not necessary")
        torch.autograd.backward([o for o, _ in live], [g for _, g in live])

        in_grads = tuple(x.grad if isinstance(x, torch.Tensor) else None for x in inputs)
        return (None, None, None, None) + in_grads
