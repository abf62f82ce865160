"""Collective front-end used by every wrapper in the library.

All FSDP / ShardedDDP / OSS / tensor-parallel / MoE code calls these functions
instead of ``torch.distributed`` directly.  Each call is routed to

* the NVLink symmetric-memory kernels (:mod:`fairscale_b200.parallel.symm`) when the
  group has a registered symmetric workspace, the tensors are CUDA tensors and
  ``FSB200_COMM`` is not ``nccl``;
* otherwise ``torch.distributed`` (NCCL on GPU — this is the "library baseline" path —
  or gloo on CPU, where missing collectives are emulated with the ones gloo has).

The reference issues the same collectives straight on c10d
(fairscale/nn/data_parallel/fully_sharded_data_parallel.py:2032-2037,
fairscale/internal/reduce_scatter_bucketer.py:38-45,145-150,
fairscale/nn/moe/moe_layer.py:29, fairscale/nn/model_parallel/mappings.py:42,76-87).
"""

from __future__ import annotations

import os
from typing import Callable, Any, List, Optional

import torch
import torch.distributed as dist

_COUNTERS = {"all_gather": 0, "reduce_scatter": 0, "all_reduce": 0, "all_to_all": 0, "broadcast": 0, "reduce": 0}


_LISTENERS: list = []


def add_listener(fn: Any) -> None:
    """Register ``fn(kind, group, out, inp)``; called before every collective issued through this module
    (``kind`` is a key of :func:`counters`).  Used by memory / traffic trackers."""
    if fn not in _LISTENERS:
        _LISTENERS.append(fn)


def remove_listener(fn: Any) -> None:
    if fn in _LISTENERS:
        _LISTENERS.remove(fn)


def _notify(kind: str, group: Any, out: Any, inp: Any) -> None:
    for fn in list(_LISTENERS):
        fn(kind, group, out, inp)


def counters() -> dict:
    """Number of collectives issued through this front-end since import (test instrumentation)."""
    return dict(_COUNTERS)


def reset_counters() -> None:
    for k in _COUNTERS:
        _COUNTERS[k] = 0


def comm_mode() -> str:
    """``"fused"`` (NVLink kernels where a workspace exists) or ``"nccl"`` (library baseline)."""
    return os.environ.get("FSB200_COMM", "fused").lower()


def group_size(group: Any) -> int:
    if group is None:
        return dist.get_world_size() if dist.is_initialized() else 1
    return group.size()


def group_rank(group: Any) -> int:
    if group is None:
        return dist.get_rank() if dist.is_initialized() else 0
    return group.rank()


def _is_real_group(group: Any) -> bool:
    """False for dummy groups used in single-process unit tests."""
    return group is None or hasattr(group, "allgather") or isinstance(group, dist.ProcessGroup)


def _backend_of(group: Any) -> str:
    try:
        return dist.get_backend(group)
    except Exception:
        return "unknown"


def _symm_for(group: Any, *tensors: torch.Tensor):
    if comm_mode() != "fused":
        return None
    if not all(t.is_cuda for t in tensors):
        return None
    from . import symm

    return symm.workspace_for(group)


def all_gather_into(out: torch.Tensor, shard: torch.Tensor, group: Any = None, async_op: bool = False):
    """``out[r*n:(r+1)*n] = shard of rank r`` for a flat ``out`` of ``world*n`` elements."""
    _COUNTERS["all_gather"] += 1
    if _LISTENERS:
        _notify("all_gather", group, out, shard)
    world = group_size(group)
    if world == 1 or not _is_real_group(group):
        out.view(-1)[: shard.numel()].copy_(shard.reshape(-1))
        return None
    ws = _symm_for(group, out, shard)
    if ws is not None and ws.can_all_gather(out, shard) and not async_op:
        ws.all_gather(out, shard)
        return None
    return dist.all_gather_into_tensor(out, shard.contiguous(), group=group, async_op=async_op)


def all_gather_last_dim(part: torch.Tensor, group: Any = None) -> torch.Tensor:
    """Every rank's ``part [..., L]`` side by side along the last dimension: ``[..., world * L]``.

    With an NVLink workspace the pulling kernel writes each rank's rows straight into their column window of the result;
    otherwise the parts are gathered along a leading axis (one collective) and moved into place by one transposing copy.
    """
    _COUNTERS["all_gather"] += 1
    world = group_size(group)
    if world == 1 or not _is_real_group(group):
        return part
    part = part.contiguous()
    out = torch.empty(*part.shape[:-1], world * part.shape[-1], dtype=part.dtype, device=part.device)
    ws = _symm_for(group, part)
    if ws is not None and ws.can_all_gather_cols(out, part):
        ws.all_gather_cols(out, part)
        return out
    stacked = torch.empty((world,) + tuple(part.shape), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(stacked.view(-1), part.view(-1), group=group)
    out.view(*part.shape[:-1], world, part.shape[-1]).copy_(stacked.movedim(0, -2))
    return out


def reduce_scatter_into(out: torch.Tensor, flat_in: torch.Tensor, group: Any = None, async_op: bool = False):
    """Sum ``flat_in`` (``world*n`` elements) over ranks; rank r keeps elements ``[r*n,(r+1)*n)``."""
    _COUNTERS["reduce_scatter"] += 1
    if _LISTENERS:
        _notify("reduce_scatter", group, out, flat_in)
    world = group_size(group)
    if world == 1 or not _is_real_group(group):
        out.copy_(flat_in.view(-1)[: out.numel()].view_as(out))
        return None
    ws = _symm_for(group, out, flat_in)
    if ws is not None and ws.can_reduce_scatter(out, flat_in) and not async_op:
        ws.reduce_scatter(out, flat_in)
        return None
    if _backend_of(group) == "gloo":
        # gloo has no reduce-scatter: all-reduce a scratch copy and keep the local slice
        tmp = flat_in.clone()
        dist.all_reduce(tmp, group=group)
        n = out.numel()
        r = group_rank(group)
        out.copy_(tmp.view(-1)[r * n : (r + 1) * n].view_as(out))
        return None
    return dist.reduce_scatter_tensor(out, flat_in.contiguous(), group=group, async_op=async_op)


def all_reduce(t: torch.Tensor, group: Any = None, op: Any = None, async_op: bool = False):
    _COUNTERS["all_reduce"] += 1
    if group_size(group) == 1 or not _is_real_group(group):
        return None
    op = dist.ReduceOp.SUM if op is None else op
    ws = _symm_for(group, t)
    if ws is not None and op == dist.ReduceOp.SUM and ws.can_all_reduce(t) and not async_op:
        ws.all_reduce(t)
        return None
    return dist.all_reduce(t, op=op, group=group, async_op=async_op)


def all_to_all_single(out: torch.Tensor, inp: torch.Tensor, group: Any = None):
    """Equal-split all-to-all over dim 0."""
    _COUNTERS["all_to_all"] += 1
    world = group_size(group)
    if world == 1 or not _is_real_group(group):
        out.copy_(inp)
        return None
    ws = _symm_for(group, out, inp)
    if ws is not None and ws.can_all_to_all(out, inp):
        ws.all_to_all(out, inp)
        return None
    if _backend_of(group) == "gloo":
        # gloo lacks all_to_all_single on some builds: emulate with all_gather
        chunks_in = list(inp.contiguous().chunk(world, dim=0))
        gathered: List[List[torch.Tensor]] = []
        r = group_rank(group)
        outs = list(out.chunk(world, dim=0))
        for src in range(world):
            bufs = [torch.empty_like(chunks_in[0]) for _ in range(world)]
            dist.all_gather(bufs, chunks_in[src], group=group)
            # bufs[k] = rank k's chunk addressed to rank `src`
            if src == r:
                for k in range(world):
                    outs[k].copy_(bufs[k])
        return None
    return dist.all_to_all_single(out, inp.contiguous(), group=group)


class StreamWork:
    """Handle of a collective that runs on a side stream of an NVLink workspace: the interface of a
    ``torch.distributed`` work object that the callers here use (``wait`` / ``is_completed``)."""

    def __init__(self, event: "torch.cuda.Event", device: torch.device) -> None:
        self.event, self.device = event, device

    def wait(self) -> bool:
        torch.cuda.current_stream(self.device).wait_event(self.event)  # stream-ordered, like a NCCL work object
        return True

    def is_completed(self) -> bool:
        return bool(self.event.query())


def _on_side_stream(ws: Any, t: torch.Tensor, fn: Callable[[], None], async_op: bool, lane: int = 3) -> Optional[StreamWork]:
    cur = torch.cuda.current_stream(t.device)
    side = ws.side_stream(lane)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        fn()
        ev = torch.cuda.Event()
        ev.record(side)
    t.record_stream(side)
    work = StreamWork(ev, t.device)
    if async_op:
        return work
    work.wait()
    return None


def _local_rank_of(group: Any, global_rank: int) -> int:
    return global_rank if group is None or group is dist.group.WORLD else dist.get_group_rank(group, global_rank)


def broadcast(t: torch.Tensor, src: int, group: Any = None, async_op: bool = False):
    """``src`` is a *global* rank, as in ``torch.distributed.broadcast``.  With an NVLink workspace the other ranks copy the
    tensor out of the owner's symmetric heap on their copy engines (OSS publishing an owner's updated parameters)."""
    _COUNTERS["broadcast"] += 1
    if group_size(group) == 1 or not _is_real_group(group):
        return None
    ws = _symm_for(group, t)
    if ws is not None and ws.can_broadcast(t):
        owner = _local_rank_of(group, src)
        return _on_side_stream(ws, t, lambda: ws.broadcast(t, owner), async_op)
    return dist.broadcast(t, src=src, group=group, async_op=async_op)


def reduce(t: torch.Tensor, dst: int, group: Any = None, async_op: bool = False):
    """Sum-reduce to the *global* rank ``dst``.  With an NVLink workspace the owner's kernel pulls the peers' buffers
    (ShardedDataParallel reducing a gradient or a gradient bucket to the rank that owns it)."""
    _COUNTERS["reduce"] += 1
    if group_size(group) == 1 or not _is_real_group(group):
        return None
    ws = _symm_for(group, t)
    if ws is not None and ws.can_reduce_to(t):
        owner = _local_rank_of(group, dst)
        return _on_side_stream(ws, t, lambda: ws.reduce_to(t, owner), async_op)
    return dist.reduce(t, dst=dst, group=group, async_op=async_op)
