"""OffloadModel: train an ``nn.Sequential`` whose parameters live in pinned host memory, one slice on the GPU at a time.

Capability parity with fairscale/experimental/nn/offload.py:39-528 (``OffloadModel(model, device,
offload_device, num_slices, checkpoint_activation, num_microbatches)``, split by parameter count, activation
checkpointing with micro-batches, profiler range names).  Design differences:

* every slice owns ONE flat pinned host buffer for its parameters and one for its gradients; a load is a
  single host-to-device copy of the flat buffer on a copy stream, and parameters are views into the device copy;
* the compute stream waits on an event recorded after the load, and a buffer is released only after an event
  recorded on the compute stream (the reference never orders its side streams against the compute stream);
* the next slice is prefetched while the current one computes (previous one in backward);
* weights are not copied back after forward (they did not change); after backward only gradients travel to the
  host, where the optimizer steps on the host parameters.
"""

from __future__ import annotations

import contextlib
import logging
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
from torch import nn
from torch.autograd.profiler import record_function

_NS = "fairscale.experimental.nn.offload:"


def _split(modules: Sequence[nn.Module], number_splits: int) -> List[List[nn.Module]]:
    """Greedy contiguous split with about equal parameter counts per slice."""
    number_splits = min(len(modules), number_splits)
    sizes = [sum(p.numel() for p in m.parameters()) for m in modules]
    per = sum(sizes) // number_splits
    splits: List[List[nn.Module]] = [[] for _ in range(number_splits)]
    cur, cur_size = 0, 0
    for m, n in zip(modules, sizes):
        if cur_size > 0 and cur_size + n > per and cur < number_splits - 1:
            cur, cur_size = cur + 1, 0
        splits[cur].append(m)
        cur_size += n
    for i, s in enumerate(splits):
        logging.info(f"Shard {i} holds {sum(p.numel() for m in s for p in m.parameters()) / 1e6:.2f}M parameters")
    return splits


class ModelShard(nn.Module):
    """One slice: host-resident flat parameter / gradient buffers and a transient device copy."""

    def __init__(self, cpu_model_shard: nn.Module, device: torch.device, offload_device: torch.device, index: int):
        super().__init__()
        self.model_shard = cpu_model_shard
        self.index = index
        self.device = torch.device(device)
        self.offload_device = torch.device(offload_device)
        self._cuda = self.device.type == "cuda"
        self.model_shard.to(self.offload_device)
        self._tensors: List[torch.Tensor] = list(self.model_shard.parameters()) + list(self.model_shard.buffers())
        self._by_dtype: dict = {}
        for t in self._tensors:
            self._by_dtype.setdefault(t.dtype, []).append(t)
        self._host: dict = {}
        self._host_grad: dict = {}
        for dt, ts in self._by_dtype.items():
            flat = torch.empty(sum(t.numel() for t in ts), dtype=dt, device=self.offload_device)
            if self._cuda and self.offload_device.type == "cpu":
                flat = flat.pin_memory()
            off = 0
            for t in ts:
                flat[off : off + t.numel()].copy_(t.detach().reshape(-1))
                t.data = flat[off : off + t.numel()].view(t.shape)
                off += t.numel()
            self._host[dt] = flat
        self._host_views = [t.data for t in self._tensors]
        self._dev: Optional[dict] = None
        self._load_event: Optional[Any] = None
        if self._cuda:
            self._cpu_to_gpu_stream = torch.cuda.Stream(device=self.device)
            self._gpu_to_cpu_stream = torch.cuda.Stream(device=self.device)

    def forward(self, *inputs: Any) -> Any:
        return self.model_shard(*inputs)

    def train(self, mode: bool = True) -> "ModelShard":
        self.model_shard.train(mode)
        return self

    def to_device(self) -> None:
        """Bring the slice onto the compute device and wait for it (the blocking form of :meth:`forward_load`)."""
        self.forward_load(non_blocking=False)
        self.use()

    @property
    def loaded(self) -> bool:
        return self._dev is not None

    # -- host -> device -------------------------------------------------------------------------------------
    def forward_load(self, non_blocking: bool = True) -> None:
        """Start copying the flat buffers to the device (no-op when already resident)."""
        if self._dev is not None:
            return
        if not self._cuda:
            self._dev = {dt: flat.clone() for dt, flat in self._host.items()}
            return
        with torch.cuda.stream(self._cpu_to_gpu_stream):
            self._dev = {dt: flat.to(self.device, non_blocking=non_blocking) for dt, flat in self._host.items()}
            self._load_event = torch.cuda.Event()
            self._load_event.record()

    backward_load = forward_load

    def use(self) -> None:
        """Point the parameters at the device copy; the current stream waits for the load."""
        self.forward_load()
        assert self._dev is not None
        if self._cuda and self._load_event is not None:
            torch.cuda.current_stream(self.device).wait_event(self._load_event)
            for flat in self._dev.values():
                flat.record_stream(torch.cuda.current_stream(self.device))
        for dt, ts in self._by_dtype.items():
            off = 0
            for t in ts:
                t.data = self._dev[dt][off : off + t.numel()].view(t.shape)
                off += t.numel()

    # -- device -> host -------------------------------------------------------------------------------------
    def forward_drop(self, non_blocking: bool = True) -> None:
        """Release the device copy.  Buffers (e.g. batch-norm statistics) may have changed and are written back;
        parameters did not change in forward."""
        if self._dev is None:
            return
        bufs = list(self.model_shard.buffers())
        n_params = len(self._tensors) - len(bufs)
        for t, host in zip(self._tensors[n_params:], self._host_views[n_params:]):
            host.copy_(t.data, non_blocking=False)
        for t, host in zip(self._tensors, self._host_views):
            t.data = host
        self._dev = None  # the caching allocator reuses the block once the recorded streams passed it

    def backward_drop(self, non_blocking: bool = True) -> None:
        """Move this slice's gradients into the host gradient buffers, then release the device copy."""
        if self._dev is None:
            return
        ev = None
        if self._cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
        for p in self.model_shard.parameters():
            if p.grad is None or p.grad.device == self.offload_device:
                continue
            g = p.grad
            host_g = getattr(p, "_host_grad", None)
            if host_g is None or host_g.shape != g.shape or host_g.dtype != g.dtype:
                host_g = torch.empty(g.shape, dtype=g.dtype, device=self.offload_device)
                if self._cuda and self.offload_device.type == "cpu":
                    host_g = host_g.pin_memory()
                p._host_grad = host_g  # type: ignore[attr-defined]
            if self._cuda:
                with torch.cuda.stream(self._gpu_to_cpu_stream):
                    self._gpu_to_cpu_stream.wait_event(ev)
                    host_g.copy_(g, non_blocking=non_blocking)
                    g.record_stream(self._gpu_to_cpu_stream)
            else:
                host_g.copy_(g)
            p.grad = None
            p._pending_host_grad = host_g  # type: ignore[attr-defined]
        self.forward_drop(non_blocking)
        for p in self.model_shard.parameters():
            pend = p.__dict__.pop("_pending_host_grad", None)
            if pend is not None:
                p.grad = pend

    def sync(self) -> None:
        """Block the host until this slice's device-to-host copies have landed (before an optimizer step on the host)."""
        if self._cuda:
            self._gpu_to_cpu_stream.synchronize()


def _to(t: Any, device: torch.device) -> Any:
    return t.to(device, non_blocking=True) if isinstance(t, torch.Tensor) else t


def _autocast_snapshot() -> Optional[Dict[str, Any]]:
    """Arguments that re-create the autocast context that is active now (None when there is none)."""
    for device_type in ("cuda", "cpu"):
        if torch.is_autocast_enabled(device_type):
            return {"device_type": device_type, "dtype": torch.get_autocast_dtype(device_type)}
    return None


class OffloadFunction(torch.autograd.Function):
    """Checkpointed execution: forward runs every slice under ``no_grad`` and keeps only the slice-boundary
    activations (on the offload device); backward reloads slices in reverse, recomputes with grad per micro-batch
    and back-propagates."""

    @staticmethod
    def forward(ctx: Any, dummy: torch.Tensor, model: "OffloadModel", *inputs: Any) -> Any:  # type: ignore[override]
        ctx.model = model
        ctx.n_inputs = len(inputs)
        ctx.autocast = _autocast_snapshot()  # the recomputation in backward runs under the autocast state of this forward
        slices = model.model_slices
        acts: List[Tuple[Any, ...]] = [tuple(inputs)]
        ctx.inputs_require_grad = [isinstance(i, torch.Tensor) and i.requires_grad for i in inputs]
        cur: Tuple[Any, ...] = tuple(inputs)
        slices[0].forward_load()
        for i, s in enumerate(slices):
            with record_function(_NS + "forward_load"):
                s.use()
                if i + 1 < len(slices):
                    slices[i + 1].forward_load()
            with record_function(_NS + "no_grad_forward_pass"), torch.no_grad():
                cur = tuple(_to(a, model.device) for a in cur)
                outs = []
                for mb in model._microbatches(cur):
                    o = s(*mb)
                    outs.append(o if isinstance(o, tuple) else (o,))
                cur = tuple(torch.cat([o[k] for o in outs]) for k in range(len(outs[0])))
            with record_function(_NS + "forward_drop"):
                s.forward_drop()
            if i + 1 < len(slices):
                acts.append(tuple(_to(a, model.offload_device) for a in cur) if model._offload_activations else cur)
        ctx.acts = acts
        out = tuple(c.detach().requires_grad_(c.is_floating_point()) if isinstance(c, torch.Tensor) else c for c in cur)
        return out[0] if len(out) == 1 else out

    @staticmethod
    def backward(ctx: Any, *grad_outputs: Any) -> Any:  # type: ignore[override]
        model: OffloadModel = ctx.model
        slices = model.model_slices
        grads: Tuple[Any, ...] = tuple(grad_outputs)
        slices[-1].backward_load()
        for i in range(len(slices) - 1, -1, -1):
            s = slices[i]
            with record_function(_NS + "backward_load"):
                s.use()
                if i > 0:
                    slices[i - 1].backward_load()
            acts = tuple(_to(a, model.device) for a in ctx.acts[i])
            in_grads: List[List[Any]] = []
            for mb, gmb in zip(model._microbatches(acts), model._microbatches(grads)):
                leaves = tuple(a.detach().requires_grad_(a.is_floating_point()) if isinstance(a, torch.Tensor) else a for a in mb)
                amp = torch.autocast(**ctx.autocast) if ctx.autocast is not None else contextlib.nullcontext()
                with record_function(_NS + "forward_pass_with_enable_grad"), torch.enable_grad(), amp:
                    o = s(*leaves)
                    o = o if isinstance(o, tuple) else (o,)
                with record_function(_NS + "backward_pass"):
                    pairs = [(a, g) for a, g in zip(o, gmb) if isinstance(a, torch.Tensor) and a.requires_grad and g is not None]
                    torch.autograd.backward([a for a, _ in pairs], [g for _, g in pairs])
                in_grads.append([l.grad if isinstance(l, torch.Tensor) else None for l in leaves])
            grads = tuple(None if in_grads[0][k] is None else torch.cat([g[k] for g in in_grads]) for k in range(len(in_grads[0])))
            with record_function(_NS + "backward_drop"):
                s.backward_drop()
        final = tuple(g if need else None for g, need in zip(grads, ctx.inputs_require_grad))
        return (None, None) + final


class ShardSyncLayer(torch.autograd.Function):
    """Boundary between slice ``index`` and ``index + 1`` when the whole graph is kept: forward drops ``index`` and
    makes ``index + 1`` resident; backward drops ``index + 1`` (with its gradients) and reloads ``index``."""

    @staticmethod
    def forward(ctx: Any, dummy: torch.Tensor, index: int, model: "OffloadModel", *inputs: Any) -> Any:  # type: ignore[override]
        slices = model.model_slices
        ctx.index, ctx.model = index, model
        if index >= 0:
            slices[index].forward_drop()
        if index + 1 < len(slices):
            slices[index + 1].use()
            if index + 2 < len(slices):
                slices[index + 2].forward_load()
        out = tuple(i.view_as(i) if isinstance(i, torch.Tensor) else i for i in inputs)
        return out[0] if len(out) == 1 else out

    @staticmethod
    def backward(ctx: Any, *grads: Any) -> Any:  # type: ignore[override]
        slices = ctx.model.model_slices
        index = ctx.index
        if index + 1 < len(slices):
            slices[index + 1].backward_drop()
        if index >= 0:
            slices[index].use()
            if index - 1 >= 0:
                slices[index - 1].backward_load()
        return (None, None, None) + tuple(grads)


class OffloadModel(nn.Module):
    """Args:
        model: ``nn.Sequential`` (split into ``num_slices`` by parameter count) or a list of modules (one slice each).
        device: compute device.  offload_device: where inactive slices live (default CPU, pinned).
        checkpoint_activation: keep only slice-boundary activations and recompute in backward.
        num_microbatches: micro-batches per slice residency (needs ``checkpoint_activation``).
        offload_activations: with checkpointing, park boundary activations on the offload device (default True,
            as the reference does; with 180 GB of HBM keeping them on the device is often the better choice).
    """

    def __init__(self, model: Any, device: torch.device, offload_device: torch.device = torch.device("cpu"),
                 num_slices: int = 3, checkpoint_activation: bool = False, num_microbatches: int = 1,
                 offload_activations: bool = True):
        super().__init__()
        if not model:
            raise TypeError("`model` argument to `OffloadModel` cannot be None.")
        if not device:
            raise TypeError("`device` argument to `OffloadModel` cannot be None.")
        if not (isinstance(model, nn.Sequential) or type(model) == list):
            raise TypeError("`model` argument to `OffloadModel` must be of type `nn.Sequential`.")
        if not checkpoint_activation and num_microbatches > 1:
            raise RuntimeError("We currently only support microbatches with activation checkpointing.")
        self.device = torch.device(device)
        self.offload_device = torch.device(offload_device)
        parts = [[m] for m in model] if type(model) == list else _split(list(model), num_slices)
        self.model_slices: List[ModelShard] = [
            ModelShard(nn.Sequential(*p) if len(p) != 1 or type(model) != list else p[0], self.device, self.offload_device, i)
            for i, p in enumerate(parts)
        ]
        self._model = nn.Sequential(*self.model_slices)
        self._checkpoint_activation = checkpoint_activation
        self._num_microbatches = num_microbatches
        self._offload_activations = offload_activations
        self._dummy = torch.zeros(1, requires_grad=True)
        if checkpoint_activation:
            # forward runs twice per step (no-grad pass + recomputation): batch-norm statistics move only once
            from ...nn.checkpoint.checkpoint_utils import patch_batchnorm

            self._bn_handles = patch_batchnorm(self._model)

    def _microbatches(self, tensors: Tuple[Any, ...]) -> List[Tuple[Any, ...]]:
        n = self._num_microbatches
        if n <= 1:
            return [tensors]
        chunks = [t.chunk(n) if isinstance(t, torch.Tensor) else [t] * n for t in tensors]
        m = min(len(c) for c in chunks)
        return [tuple(c[i] for c in chunks) for i in range(m)]

    def sync(self) -> None:
        """Wait until every gradient has reached the host (call before ``optimizer.step()``; ``forward`` of the
        next step does it implicitly)."""
        for s in self.model_slices:
            s.sync()

    def forward(self, *inputs: Any, **_: Any) -> Any:  # type: ignore[override]
        self.sync()
        if self._checkpoint_activation:
            return OffloadFunction.apply(self._dummy, self, *inputs)
        cur: Any = tuple(_to(i, self.device) for i in inputs)
        self.model_slices[0].forward_load()
        for index in range(-1, len(self.model_slices)):
            if index >= 0:
                cur = self.model_slices[index](*cur)
                cur = cur if isinstance(cur, tuple) else (cur,)
            cur = ShardSyncLayer.apply(self._dummy, index, self, *cur)
            cur = cur if isinstance(cur, tuple) else (cur,)
        return cur[0] if len(cur) == 1 else cur
