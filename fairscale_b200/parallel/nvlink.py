"""NVLink symmetric-memory workspace: the Python side of ``csrc/comm.cu``.

``enable(group)`` allocates, once per process group, a symmetric heap (peer-mapped by every rank of the
group through ``torch.distributed._symmetric_memory`` — the rendezvous is plain torch.distributed plumbing)
plus a signal pad, and registers a :class:`NvlinkWorkspace` so that :mod:`fairscale_b200.parallel.comm`
routes FSDP / tensor-parallel / MoE collectives to the in-kernel NVLink implementations.

A tensor that already lives in the heap is used in place; any other tensor is first copied into a staging
area of the heap (a local HBM copy, ~10x cheaper than the NVLink transfer it feeds).  Independent "lanes"
(own staging, channels and epoch counters) let collectives run concurrently on different streams, e.g. FSDP's
all-gather stream and its gradient-reduction stream.
"""

from __future__ import annotations

import ctypes
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native
from ..ops import _bind
from . import symm

_SIGS_DONE = False


def _sigs() -> None:
    global _SIGS_DONE
    if _SIGS_DONE:
        return
    from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

    head = [c_int, c_int, c_uint, c_int, c_void_p]
    S = _bind._SIGNATURES
    S["fsb_comm_barrier"] = head + [c_void_p, c_void_p]
    S["fsb_comm_all_gather"] = head + [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p]
    S["fsb_comm_all_to_all"] = head + [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p]
    S["fsb_comm_reduce_scatter"] = head + [c_void_p, c_void_p, c_int, c_void_p, c_int, c_longlong, c_float, c_int, c_void_p, c_void_p]
    S["fsb_comm_all_reduce"] = head + [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p]
    S["fsb_comm_moe_scatter_rows"] = head + [c_void_p] * 6 + [c_longlong, c_int, c_int, c_void_p, c_void_p]
    S["fsb_comm_moe_gather_rows"] = head + [c_void_p] * 8 + [c_longlong, c_int, c_int, c_void_p, c_void_p]
    _SIGS_DONE = True


def _ptr_array(ptrs: List[int]) -> Any:
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


class _Lane:
    """Staging window + channels + epochs for one stream of collectives."""

    def __init__(self, index: int, staging_off: int, staging_bytes: int):
        self.index = index
        self.staging_off = staging_off
        self.staging_bytes = staging_bytes
        self.epoch = 0
        self.channel = index * 4  # each lane owns 4 consecutive channels


class NvlinkWorkspace:
    N_LANES = 4

    def __init__(self, group: Any, device: torch.device, staging_mb: int = 256, heap_mb: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        _sigs()
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > _bind.fn("fsb_comm_max_ranks")():
            raise ValueError("NVLink workspace supports up to 8 ranks (one NVSwitch domain)")
        self.device = device
        staging = staging_mb << 20
        self.heap_bytes = self.N_LANES * staging + (heap_mb << 20)
        self.heap = symm_mem.empty(self.heap_bytes, dtype=torch.uint8, device=device)
        self.heap_handle = symm_mem.rendezvous(self.heap, self.group)
        self.peer_base: List[int] = [int(p) for p in self.heap_handle.buffer_ptrs]
        self.pads = symm_mem.empty(64 * 8, dtype=torch.int32, device=device)
        self.pads.zero_()
        self.pads_handle = symm_mem.rendezvous(self.pads, self.group)
        self.pad_ptrs = _ptr_array([int(p) for p in self.pads_handle.buffer_ptrs])
        self.counters = torch.zeros(64, dtype=torch.int32, device=device)
        self.lanes = [_Lane(i, i * staging, staging) for i in range(self.N_LANES)]
        self._bump = self.N_LANES * staging
        self.base = self.heap.data_ptr()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # pads are zero everywhere before the first kernel signals

    # ------------------------------------------------------------------ heap
    def alloc(self, nbytes: int, align: int = 256) -> torch.Tensor:
        """Persistent uint8 window of the symmetric heap (same offset on every rank when called collectively)."""
        off = (self._bump + align - 1) // align * align
        if off + nbytes > self.heap_bytes:
            raise MemoryError("symmetric heap exhausted; pass a larger heap_mb to nvlink.enable()")
        self._bump = off + nbytes
        return self.heap[off : off + nbytes]

    def scratch(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Named, reusable heap tensor (allocated on first use; the same name and size returns the same window)."""
        key = (name, tuple(shape), dtype)
        cache = self.__dict__.setdefault("_scratch", {})
        if key not in cache:
            cache[key] = self.alloc_tensor(tuple(shape), dtype)
        return cache[key]

    def alloc_tensor(self, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        return self.alloc(n * torch.empty((), dtype=dtype).element_size()).view(dtype).view(shape)

    def offset_of(self, t: torch.Tensor) -> Optional[int]:
        off = t.data_ptr() - self.base
        if 0 <= off and off + t.numel() * t.element_size() <= self.heap_bytes:
            return off
        return None

    def peers(self, offset: int) -> Any:
        return _ptr_array([b + offset for b in self.peer_base])

    def _stage(self, lane: _Lane, t: torch.Tensor, total_bytes: Optional[int] = None) -> int:
        """Copy ``t`` into the lane's staging window (zero-padding up to ``total_bytes``); returns its heap offset."""
        nbytes = t.numel() * t.element_size()
        total = total_bytes or nbytes
        if total > lane.staging_bytes:
            raise MemoryError("tensor larger than the staging window; enable() with a larger staging_mb")
        window = self.heap[lane.staging_off : lane.staging_off + total]
        window[:nbytes].view(t.dtype).copy_(t.reshape(-1))
        if total > nbytes:
            window[nbytes:].zero_()
        return lane.staging_off

    def _head(self, lane: _Lane) -> tuple:
        lane.epoch = (lane.epoch + 1) & 0x7FFFFFFF
        return (self.rank, self.world, lane.epoch, lane.channel, self.pad_ptrs)

    def _counter(self, lane: _Lane) -> int:
        return self.counters.data_ptr() + 4 * lane.index

    def _lane(self, lane: int) -> _Lane:
        return self.lanes[lane % self.N_LANES]

    # ------------------------------------------------------------------ capability checks used by comm.py
    def _fits(self, t: torch.Tensor, nbytes: int) -> bool:
        """A tensor outside the symmetric heap is copied into a lane's staging window first and has to fit there."""
        return self.offset_of(t) is not None or nbytes <= self.lanes[0].staging_bytes

    def can_all_gather(self, out: torch.Tensor, shard: torch.Tensor) -> bool:
        nbytes = shard.numel() * shard.element_size()
        return out.is_contiguous() and nbytes % 16 == 0 and out.numel() == shard.numel() * self.world and self._fits(shard, nbytes)

    def can_reduce_scatter(self, out: torch.Tensor, flat_in: torch.Tensor) -> bool:
        if not (flat_in.dtype in _bind._DTYPE_CODE and out.dtype in _bind._DTYPE_CODE and (out.numel() * flat_in.element_size()) % 16 == 0):
            return False
        need = out.numel() * self.world * flat_in.element_size()
        in_heap = self.offset_of(flat_in) is not None and flat_in.numel() == out.numel() * self.world
        return in_heap or need <= self.lanes[0].staging_bytes

    def can_all_reduce(self, t: torch.Tensor) -> bool:
        return t.dtype in _bind._DTYPE_CODE and t.is_contiguous() and self._fits(t, t.numel() * t.element_size())

    def can_all_to_all(self, out: torch.Tensor, inp: torch.Tensor) -> bool:
        nbytes = inp.numel() * inp.element_size()
        return inp.is_contiguous() and out.is_contiguous() and (nbytes // self.world) % 16 == 0 and self._fits(inp, nbytes)

    # ------------------------------------------------------------------ collectives
    def barrier(self, lane: int = 0) -> None:
        ln = self._lane(lane)
        _bind.call("fsb_comm_barrier", *self._head(ln), _bind.status_ptr(self.device), _bind.stream_ptr(self.device))

    def all_gather(self, out: torch.Tensor, shard: torch.Tensor, lane: int = 1) -> None:
        ln = self._lane(lane)
        shard = shard.contiguous()
        off = self.offset_of(shard)
        if off is None:
            off = self._stage(ln, shard)
        _bind.call("fsb_comm_all_gather", *self._head(ln), self._counter(ln), self.peers(off), out.data_ptr(),
                   shard.numel() * shard.element_size(), _bind.status_ptr(self.device), _bind.stream_ptr(self.device))

    def reduce_scatter(self, out: torch.Tensor, flat_in: torch.Tensor, scale: float = 1.0, accumulate: bool = False, lane: int = 2) -> None:
        """``out = (out if accumulate else 0) + scale * sum_ranks flat_in[rank * n : (rank + 1) * n]``, n = out.numel();
        ``flat_in`` may be shorter than ``world * n`` (implicit zero padding)."""
        ln = self._lane(lane)
        n = out.numel()
        flat_in = flat_in.contiguous()
        need = n * self.world * flat_in.element_size()
        off = self.offset_of(flat_in)
        if off is None or flat_in.numel() != n * self.world:
            off = self._stage(ln, flat_in, need)
        _bind.call("fsb_comm_reduce_scatter", *self._head(ln), self._counter(ln), self.peers(off), _bind.dtype_code(flat_in.dtype),
                   out.data_ptr(), _bind.dtype_code(out.dtype), n, scale, int(accumulate), _bind.status_ptr(self.device),
                   _bind.stream_ptr(self.device))

    def all_reduce(self, t: torch.Tensor, lane: int = 0) -> None:
        ln = self._lane(lane)
        off = self.offset_of(t)
        staged = off is None
        if staged:
            off = self._stage(ln, t)
        _bind.call("fsb_comm_all_reduce", *self._head(ln), self._counter(ln), self.peers(off), _bind.dtype_code(t.dtype), t.numel(),
                   _bind.status_ptr(self.device), _bind.stream_ptr(self.device))
        if staged:
            nbytes = t.numel() * t.element_size()
            t.view(-1).copy_(self.heap[off : off + nbytes].view(t.dtype))

    def all_to_all(self, out: torch.Tensor, inp: torch.Tensor, lane: int = 0) -> None:
        ln = self._lane(lane)
        off = self.offset_of(inp)
        if off is None:
            off = self._stage(ln, inp)
        chunk_bytes = inp.numel() * inp.element_size() // self.world
        _bind.call("fsb_comm_all_to_all", *self._head(ln), self._counter(ln), self.peers(off), out.data_ptr(), chunk_bytes,
                   _bind.status_ptr(self.device), _bind.stream_ptr(self.device))

    # ------------------------------------------------------------------ MoE routing (see nn/moe/moe_layer.py)
    def moe_scatter_rows(self, dst: torch.Tensor, x: torch.Tensor, dst_rank: torch.Tensor, dst_row: torch.Tensor,
                         weights: Optional[torch.Tensor], rows_per_token: int, lane: int = 0) -> None:
        """Store row ``t // rows_per_token`` of ``x`` into row ``dst_row[t]`` of rank ``dst_rank[t]``'s ``dst`` (heap tensor)."""
        ln = self._lane(lane)
        off = self.offset_of(dst)
        assert off is not None, "destination must live in the symmetric heap"
        _bind.call("fsb_comm_moe_scatter_rows", *self._head(ln), self._counter(ln), self.peers(off), x.data_ptr(), dst_rank.data_ptr(),
                   dst_row.data_ptr(), _bind.ptr(weights), dst_rank.numel(), rows_per_token, x.shape[-1],
                   _bind.status_ptr(self.device), _bind.stream_ptr(self.device))

    def moe_gather_rows(self, src: torch.Tensor, out: Optional[torch.Tensor], src_rank: torch.Tensor, src_row: torch.Tensor,
                        weights: Optional[torch.Tensor], rows_per_token: int, grad: Optional[torch.Tensor] = None,
                        dots: Optional[torch.Tensor] = None, lane: int = 0) -> None:
        ln = self._lane(lane)
        off = self.offset_of(src)
        assert off is not None, "source must live in the symmetric heap"
        tokens = src_rank.numel() // rows_per_token
        _bind.call("fsb_comm_moe_gather_rows", *self._head(ln), self._counter(ln), self.peers(off), _bind.ptr(out), src_rank.data_ptr(),
                   src_row.data_ptr(), _bind.ptr(weights), _bind.ptr(grad), _bind.ptr(dots), tokens, rows_per_token, src.shape[-1],
                   _bind.status_ptr(self.device), _bind.stream_ptr(self.device))


def enable(group: Any = None, device: Optional[torch.device] = None, staging_mb: int = 256, heap_mb: int = 0) -> NvlinkWorkspace:
    """Create (collectively) and register the NVLink workspace of ``group``; returns it."""
    group = group if group is not None else dist.group.WORLD
    existing = symm.workspace_for(group)
    if existing is not None:
        return existing
    device = device or torch.device("cuda", torch.cuda.current_device())
    ws = NvlinkWorkspace(group, device, staging_mb=staging_mb, heap_mb=heap_mb)
    symm.register_workspace(group, ws)
    return ws


def available() -> bool:
    """True when the native library is present and torch exposes symmetric memory on this build."""
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return _native.available() and torch.cuda.is_available() and torch.cuda.device_count() > 1
