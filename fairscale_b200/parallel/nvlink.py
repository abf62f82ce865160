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
import os
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
    S["fsb_comm_set_timeout_ms"] = [c_longlong]
    S["fsb_comm_barrier"] = head + [c_void_p, c_void_p]
    S["fsb_comm_all_gather"] = head + [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p]
    S["fsb_comm_gather_ranges_dma"] = head + [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    S["fsb_comm_all_gather_cols"] = head + [c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p]
    S["fsb_comm_all_gather_dma"] = head + [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p]
    S["fsb_comm_gather_flagged_copies"] = [c_int, c_int, c_int, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_longlong, c_int,
                                           c_void_p, c_uint, c_void_p]
    S["fsb_comm_gather_blocks_flagged"] = [c_int, c_int, c_int, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_uint, c_void_p]
    S["fsb_comm_all_to_all"] = head + [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p]
    S["fsb_comm_reduce_scatter"] = head + [c_void_p, c_void_p, c_int, c_void_p, c_int, c_longlong, c_float, c_int, c_void_p, c_void_p]
    S["fsb_comm_reduce_scatter_dma"] = head + [c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_float, c_int, c_void_p, c_void_p]
    S["fsb_comm_reduce_scatter_adam"] = head + [c_void_p, c_void_p, c_int, c_longlong, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_float, c_float, c_float, c_float, c_float, c_float, c_int, c_int, c_void_p, c_void_p,
                                                 c_void_p, c_void_p]
    S["fsb_comm_reduce_to"] = head + [c_void_p, c_void_p, c_int, c_longlong, c_float, c_int, c_void_p, c_void_p]
    S["fsb_comm_broadcast_dma"] = head + [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p]
    S["fsb_comm_all_reduce"] = head + [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p]
    S["fsb_comm_moe_scatter_rows"] = head + [c_void_p] * 6 + [c_longlong, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
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
    DMA_MIN_BYTES = 1 << 20  # below this the extra enqueues of the copy-engine all-gather cost more than they save

    def __init__(self, group: Any, device: torch.device, staging_mb: int = 256, heap_mb: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        _sigs()
        if os.environ.get("FSB200_COMM_TIMEOUT_S"):
            set_timeout(float(os.environ["FSB200_COMM_TIMEOUT_S"]))
        self._peer_cache: Dict[int, Any] = {}
        # "kernel": one kernel pulls the shards with SM-issued loads; "dma": copy engines move them between two flag barriers
        self.all_gather_engine = os.environ.get("FSB200_AG", "dma").lower()
        self.reduce_scatter_engine = os.environ.get("FSB200_RS", "dma").lower()  # "dma": copy engines + local sum; "kernel": pull kernel
        self._rs_stage: Dict[int, torch.Tensor] = {}  # per lane: landing buffer of the peers' slices
        self.poisoned = False  # set when a kernel gave up a wait: flags and epochs can no longer be trusted
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
        guards = self._guards()
        taken = nbytes if guards is None else guards.reserve(nbytes)
        if off + taken > self.heap_bytes:
            raise MemoryError("symmetric heap exhausted; pass a larger heap_mb to nvlink.enable()")
        self._bump = off + taken
        if guards is not None:
            guards.plant(off, nbytes)
        return self.heap[off : off + nbytes]

    def _guards(self) -> Optional[Any]:
        """Guard words behind every heap window when ``FSB200_HEAP_CANARY=1`` (see :mod:`fairscale_b200.parallel.heap_guard`)."""
        from . import heap_guard

        if not heap_guard.enabled():
            return None
        if getattr(self, "_heap_guards", None) is None:
            self._heap_guards = heap_guard.HeapGuards(self.heap)
        return self._heap_guards

    def check_canaries(self) -> None:
        """Raise if a guard behind a heap window was overwritten (debug aid; synchronises the device).  A no-op unless the
        workspace was created with ``FSB200_HEAP_CANARY=1``."""
        guards = getattr(self, "_heap_guards", None)
        if guards is None:
            return
        torch.cuda.synchronize(self.device)
        bad = guards.corrupted()
        if bad:
            guards.replant()
            raise RuntimeError("symmetric heap overrun on rank %d:\n  " % self.rank + "\n  ".join(bad))

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
        window = self.alloc(n * torch.empty((), dtype=dtype).element_size())
        # A tensor of its own on the heap's storage, not a view of the heap tensor: in-place operations on one window must
        # not count as modifications of every other window (autograd refuses custom-Function outputs whose base changed).
        esize = torch.empty((), dtype=dtype).element_size()
        t = torch.empty(0, dtype=dtype, device=self.device)
        t.set_(self.heap.untyped_storage(), (window.data_ptr() - self.heap.data_ptr() + self.heap.storage_offset()) // esize, tuple(shape))
        return t

    # ------------------------------------------------------------------ gradient windows
    def enable_grad_windows(self, window_bytes: int, count: int = 3) -> None:
        """Reserve ``count`` equal windows of the heap (collectively: same offsets on every rank) that :meth:`grad_window`
        hands out in rotation as flat-gradient buffers.  A gradient produced there is reduce-scattered in place: the
        peers' kernels read it where the weight-gradient GEMMs wrote it."""
        if getattr(self, "_gw_offsets", None):
            return
        window_bytes = (window_bytes + 255) // 256 * 256
        self._gw_bytes = window_bytes
        self._gw_offsets = []
        for _ in range(count):
            w = self.alloc(window_bytes)
            self._gw_offsets.append(w.data_ptr() - self.base)
        self._gw_next = 0
        self._gw_busy: Dict[int, Any] = {}

    def grad_window(self, numel: int, dtype: torch.dtype, device: torch.device) -> Optional[torch.Tensor]:
        """Next gradient window as a ``numel``-element tensor (None if windows are off or too small).  The elements up to
        the next multiple of the world size (the implicit padding of a reduce-scatter) are zeroed.  The current stream
        first waits until the previous user of the window (a reduce-scatter, hence also every peer's reads) is done."""
        offs = getattr(self, "_gw_offsets", None)
        esize = torch.empty((), dtype=dtype).element_size()
        pad = 2 * self.world + 16
        if not offs or self.poisoned or device != self.device or (numel + pad) * esize > self._gw_bytes:
            return None
        off = offs[self._gw_next]
        self._gw_next = (self._gw_next + 1) % len(offs)
        busy = self._gw_busy.pop(off, None)
        if busy is not None:
            torch.cuda.current_stream(self.device).wait_event(busy)
        buf = self.heap[off : off + (numel + pad) * esize].view(dtype)
        buf[numel:].zero_()
        return buf[:numel]

    def _window_of(self, t: torch.Tensor) -> Optional[int]:
        offs = getattr(self, "_gw_offsets", None)
        if not offs:
            return None
        off = t.data_ptr() - self.base
        return off if off in offs else None

    def release_grad_window(self, t: torch.Tensor) -> None:
        """Note that the launches enqueued so far on the current stream are the last readers of gradient window ``t``."""
        off = self._window_of(t)
        if off is not None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._gw_busy[off] = ev

    def offset_of(self, t: torch.Tensor) -> Optional[int]:
        off = t.data_ptr() - self.base
        if 0 <= off and off + t.numel() * t.element_size() <= self.heap_bytes:
            return off
        return None

    def peers(self, offset: int) -> Any:
        """ctypes array with the address of heap offset ``offset`` on every rank (cached: the offsets of persistent
        shards and staging windows repeat every step)."""
        arr = self._peer_cache.get(offset)
        if arr is None:
            if len(self._peer_cache) > 4096:
                self._peer_cache.clear()
            arr = self._peer_cache[offset] = _ptr_array([b + offset for b in self.peer_base])
        return arr

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

    @staticmethod
    def _aligned(*tensors: torch.Tensor) -> bool:
        """The kernels move 16-byte vectors: every CUDA pointer they get must sit on a 16-byte boundary."""
        return all(t.is_cuda and t.data_ptr() % 16 == 0 for t in tensors)

    def can_all_gather(self, out: torch.Tensor, shard: torch.Tensor) -> bool:
        nbytes = shard.numel() * shard.element_size()
        return (out.is_contiguous() and nbytes % 16 == 0 and out.numel() == shard.numel() * self.world and self._fits(shard, nbytes)
                and self._aligned(out) and (self.offset_of(shard) is None or self._aligned(shard)))

    def can_reduce_scatter(self, out: torch.Tensor, flat_in: torch.Tensor) -> bool:
        if not (flat_in.dtype in _bind._DTYPE_CODE and out.dtype in _bind._DTYPE_CODE and (out.numel() * flat_in.element_size()) % 16 == 0):
            return False
        if not (self._aligned(out) and flat_in.is_cuda and out.is_contiguous()):
            return False  # e.g. a host-resident master shard (CPU offload): the kernel writes `out` directly
        need = out.numel() * self.world * flat_in.element_size()
        in_heap = self.offset_of(flat_in) is not None and (flat_in.numel() == out.numel() * self.world or self._window_of(flat_in) is not None)
        return (in_heap and self._aligned(flat_in)) or need <= self.lanes[0].staging_bytes

    def can_all_reduce(self, t: torch.Tensor) -> bool:
        return (t.dtype in _bind._DTYPE_CODE and t.is_contiguous() and self._fits(t, t.numel() * t.element_size())
                and (self.offset_of(t) is None or self._aligned(t)))

    def can_all_to_all(self, out: torch.Tensor, inp: torch.Tensor) -> bool:
        nbytes = inp.numel() * inp.element_size()
        return (inp.is_contiguous() and out.is_contiguous() and (nbytes // self.world) % 16 == 0 and self._fits(inp, nbytes)
                and self._aligned(out) and (self.offset_of(inp) is None or self._aligned(inp)))

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
        nbytes = shard.numel() * shard.element_size()
        if self.all_gather_engine == "dma" and nbytes >= self.DMA_MIN_BYTES:
            # payload on the copy engines (no SM takes part): two flag barriers around one peer copy per rank
            head = self._head(ln)
            ln.epoch = (ln.epoch + 1) & 0x7FFFFFFF  # the exit barrier uses the next epoch
            _bind.call("fsb_comm_all_gather_dma", *head, self.peers(off), out.data_ptr(), nbytes, _bind.status_ptr(self.device),
                       _bind.stream_ptr(self.device), launches=2)
            return
        _bind.call("fsb_comm_all_gather", *self._head(ln), self._counter(ln), self.peers(off), out.data_ptr(),
                   nbytes, _bind.status_ptr(self.device), _bind.stream_ptr(self.device))

    def barrier_on(self, channel: int, epoch: int) -> None:
        """Flag barrier on an explicit signal-pad channel (callers outside the collective lanes keep their own epochs)."""
        _bind.call("fsb_comm_barrier", self.rank, self.world, epoch, channel, self.pad_ptrs, _bind.status_ptr(self.device),
                   _bind.stream_ptr(self.device))

    def gather_flagged_copies(self, out: torch.Tensor, shard: torch.Tensor, first: Tuple[int, int], piece_bytes: int,
                              flags: torch.Tensor, flag_value: int, phase: int, first_piece: int = 0) -> None:
        """The copies of an all-gather of heap-resident ``shard`` into ``out``, reporting progress: elements
        ``first = [lo, hi)`` of ``out`` go first, in pieces of ``piece_bytes``, and ``flags[i] = flag_value`` is stored by
        the driver (in stream order) once the ``i``-th piece sent is in place (pieces go out cyclically from ``first_piece``
        on); the rest follows.  ``phase=0`` (on the consumer's
        stream, before the consumer) copies this rank's own part of ``first``; ``phase=1`` (on a side stream that waits
        for phase 0) moves the peers' parts on the copy engines and stores the flags, then the remainder.  No kernel is
        launched, and nothing a persistent consumer waits for needs an SM.  The caller provides the barriers around the
        two calls (:func:`fairscale_b200.parallel.fused_tp.weight_gather_gemm`)."""
        off = self.offset_of(shard)
        assert off is not None, "the shard must live in the symmetric heap"
        es = shard.element_size()
        n_pieces = -(-(first[1] - first[0]) * es // piece_bytes)
        assert flags.dtype == torch.int32 and flags.numel() >= n_pieces
        _bind.call("fsb_comm_gather_flagged_copies", self.rank, self.world, phase, self.peers(off), out.data_ptr(), shard.numel() * es, first[0] * es,
                   first[1] * es, piece_bytes, first_piece, flags.data_ptr(), flag_value, _bind.stream_ptr(self.device), launches=0)

    def gather_blocks_flagged(self, out: torch.Tensor, block: torch.Tensor, piece_bytes: int, flags: torch.Tensor, flag_value: int,
                              phase: int) -> None:
        """The copies of an all-gather of equal blocks (``out`` = the ranks' heap-resident ``block``s in rank order), reporting
        progress: blocks arrive this rank's own first, then rank + 1, ... cyclically, in pieces of ``piece_bytes``, and
        ``flags[k * pieces_per_block + j] = flag_value`` is stored by the driver once piece ``j`` of the k-th arriving block
        is in place.  ``phase=0`` (consumer's stream): own block; ``phase=1`` (side stream waiting for phase 0): the peers'
        blocks on the copy engines.  See :meth:`gather_flagged_copies` for why, and for who provides the barriers."""
        off = self.offset_of(block)
        assert off is not None, "the block must live in the symmetric heap"
        nbytes = block.numel() * block.element_size()
        assert flags.dtype == torch.int32 and flags.numel() >= self.world * -(-nbytes // piece_bytes)
        _bind.call("fsb_comm_gather_blocks_flagged", self.rank, self.world, phase, self.peers(off), out.data_ptr(), nbytes, piece_bytes,
                   flags.data_ptr(), flag_value, _bind.stream_ptr(self.device), launches=0)

    def gather_ranges(self, out: torch.Tensor, shard: torch.Tensor, ranges: List[Tuple[int, int]], lane: int = 1) -> None:
        """Fetch only the element ranges ``[lo, hi)`` of the gathered flat buffer ``out`` (the shards' concatenation) from
        the shards that hold them, on the copy engines.  Used for the small parameters a unit needs before the kernel
        that gathers the rest; that kernel's exit barrier also covers these reads."""
        ln = self._lane(lane)
        off = self.offset_of(shard)
        assert off is not None, "the shard must live in the symmetric heap"
        es = shard.element_size()
        lo = (ctypes.c_longlong * len(ranges))(*[a * es for a, _ in ranges])
        hi = (ctypes.c_longlong * len(ranges))(*[b * es for _, b in ranges])
        _bind.call("fsb_comm_gather_ranges_dma", *self._head(ln), self.peers(off), out.data_ptr(), shard.numel() * es, len(ranges),
                   lo, hi, _bind.status_ptr(self.device), _bind.stream_ptr(self.device))

    def can_all_gather_cols(self, out: torch.Tensor, part: torch.Tensor) -> bool:
        row_bytes = part.shape[-1] * part.element_size()
        return (part.dim() >= 1 and part.is_contiguous() and out.is_contiguous() and row_bytes % 16 == 0 and self._aligned(out)
                and out.numel() == part.numel() * self.world and self._fits(part, part.numel() * part.element_size())
                and (self.offset_of(part) is None or self._aligned(part)))

    def all_gather_cols(self, out: torch.Tensor, part: torch.Tensor, lane: int = 0) -> None:
        """``out[..., r * L:(r + 1) * L] = part of rank r`` (L = ``part.shape[-1]``): a gather along the last dimension
        written straight into its interleaved layout by the pulling kernel."""
        ln = self._lane(lane)
        off = self.offset_of(part)
        if off is None:
            off = self._stage(ln, part)
        rows = part.numel() // part.shape[-1]
        _bind.call("fsb_comm_all_gather_cols", *self._head(ln), self._counter(ln), self.peers(off), out.data_ptr(), rows,
                   part.shape[-1] * part.element_size(), _bind.status_ptr(self.device), _bind.stream_ptr(self.device))

    def reduce_scatter(self, out: torch.Tensor, flat_in: torch.Tensor, scale: float = 1.0, accumulate: bool = False, lane: int = 2) -> None:
        """``out = (out if accumulate else 0) + scale * sum_ranks flat_in[rank * n : (rank + 1) * n]``, n = out.numel();
        ``flat_in`` may be shorter than ``world * n`` (implicit zero padding)."""
        ln = self._lane(lane)
        n = out.numel()
        flat_in = flat_in.contiguous()
        need = n * self.world * flat_in.element_size()
        off = self.offset_of(flat_in)
        window = self._window_of(flat_in) if off is not None else None
        if off is None or (flat_in.numel() != n * self.world and (window is None or need > self._gw_bytes)):
            off = self._stage(ln, flat_in, need)  # local copy into the lane's staging window (zero padded)
        es = flat_in.element_size()
        if self.reduce_scatter_engine == "dma" and self.world > 1 and n * es >= self.DMA_MIN_BYTES:
            # the peers' copies of this rank's slice travel on the copy engines (no SM takes part) between two flag
            # barriers; a short local kernel then sums them in rank order
            stage = self._rs_stage.get(ln.index)
            want = (self.world - 1) * n * es
            if stage is None or stage.numel() < want:
                stage = self._rs_stage[ln.index] = torch.empty(want, dtype=torch.uint8, device=self.device)
            head = self._head(ln)
            ln.epoch = (ln.epoch + 1) & 0x7FFFFFFF  # the exit barrier uses the next epoch
            _bind.call("fsb_comm_reduce_scatter_dma", *head, self.peers(off), _bind.dtype_code(flat_in.dtype), stage.data_ptr(),
                       out.data_ptr(), _bind.dtype_code(out.dtype), n, scale, int(accumulate), _bind.status_ptr(self.device),
                       _bind.stream_ptr(self.device), launches=3)
            stage.record_stream(torch.cuda.current_stream(self.device))
        else:
            _bind.call("fsb_comm_reduce_scatter", *self._head(ln), self._counter(ln), self.peers(off), _bind.dtype_code(flat_in.dtype),
                       out.data_ptr(), _bind.dtype_code(out.dtype), n, scale, int(accumulate), _bind.status_ptr(self.device),
                       _bind.stream_ptr(self.device))
        if window is not None:
            self.release_grad_window(flat_in)  # the kernel's exit barrier covers the peers' reads of this window

    def can_reduce_scatter_adam(self, flat_in: torch.Tensor, p: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
                                p_copy: Optional[torch.Tensor]) -> bool:
        """The fused reduce-scatter + Adam kernel reads the flat gradient where it lies, so that has to be a gradient
        window of the heap; master parameter and moments are fp32 shards on this device."""
        n = p.numel()
        return (self._window_of(flat_in) is not None and flat_in.dtype in (torch.bfloat16, torch.float16, torch.float32)
                and (n * flat_in.element_size()) % 16 == 0 and n * self.world * flat_in.element_size() <= self._gw_bytes
                and all(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n for t in (p, m, v)) and self._aligned(p, m, v)
                and (p_copy is None or (p_copy.dtype in (torch.bfloat16, torch.float16) and p_copy.numel() == n and p_copy.data_ptr() % 8 == 0)))

    def reduce_scatter_adam(self, flat_in: torch.Tensor, p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, p_copy: Optional[torch.Tensor],
                            scale: float, step_size: float, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
                            eps_inside_sqrt: bool, adamw: bool, gnorm_sq: Optional[torch.Tensor] = None,
                            found_inf: Optional[torch.Tensor] = None, lane: int = 2) -> None:
        """One kernel: ``g = scale * sum_ranks flat_in[rank slice]`` and the Adam update of ``p, m, v`` with it; the updated
        value also goes to ``p_copy`` (the compute-dtype shard the next all-gather reads)."""
        ln = self._lane(lane)
        off = self.offset_of(flat_in)
        assert off is not None and self._window_of(flat_in) is not None
        _bind.call("fsb_comm_reduce_scatter_adam", *self._head(ln), self._counter(ln), self.peers(off), _bind.dtype_code(flat_in.dtype),
                   p.numel(), scale, p.data_ptr(), m.data_ptr(), v.data_ptr(), _bind.ptr(p_copy),
                   _bind.dtype_code(p_copy.dtype) if p_copy is not None else 0, step_size, lr, beta1, beta2, eps, weight_decay,
                   int(eps_inside_sqrt), int(adamw), _bind.ptr(gnorm_sq), _bind.ptr(found_inf), _bind.status_ptr(self.device),
                   _bind.stream_ptr(self.device))
        self.release_grad_window(flat_in)

    # ------------------------------------------------------------------ one-owner collectives (ZeRO-1 / ZeRO-2)
    def side_stream(self, lane: int) -> "torch.cuda.Stream":
        """The stream on which the collectives of ``lane`` run when they are to overlap with the caller's stream."""
        streams = self.__dict__.setdefault("_side_streams", {})
        if lane not in streams:
            streams[lane] = torch.cuda.Stream(device=self.device)
        return streams[lane]

    def can_reduce_to(self, t: torch.Tensor) -> bool:
        return (t.is_cuda and t.dtype in _bind._DTYPE_CODE and t.is_contiguous() and not self.poisoned
                and self._fits(t, t.numel() * t.element_size()) and (self.offset_of(t) is None or self._aligned(t)))

    def reduce_to(self, t: torch.Tensor, owner: int, scale: float = 1.0, lane: int = 3) -> None:
        """Sum of every rank's ``t`` into rank ``owner``'s ``t`` (in place, times ``scale``); the other ranks keep theirs.
        The owner's kernel pulls from the peers' heap (a tensor outside the heap is staged first, on every rank alike)."""
        ln = self._lane(lane)
        off = self.offset_of(t)
        staged = off is None
        if staged:
            off = self._stage(ln, t)
        _bind.call("fsb_comm_reduce_to", *self._head(ln), self._counter(ln), self.peers(off), _bind.dtype_code(t.dtype), t.numel(), scale,
                   owner, _bind.status_ptr(self.device), _bind.stream_ptr(self.device))
        if staged and owner == self.rank:
            t.view(-1).copy_(self.heap[off : off + t.numel() * t.element_size()].view(t.dtype))

    def can_broadcast(self, t: torch.Tensor) -> bool:
        return t.is_cuda and t.is_contiguous() and not self.poisoned and self._fits(t, t.numel() * t.element_size())

    def broadcast(self, t: torch.Tensor, owner: int, lane: int = 3) -> None:
        """Every rank's ``t`` becomes rank ``owner``'s: the others copy it out of the owner's heap on their copy engines
        (no SM takes part).  Whether ``t`` lives in the heap must be the same on every rank."""
        ln = self._lane(lane)
        off = self.offset_of(t)
        if off is None:
            off = self._stage(ln, t) if owner == self.rank else ln.staging_off
        head = self._head(ln)
        ln.epoch = (ln.epoch + 1) & 0x7FFFFFFF  # the exit barrier uses the next epoch
        _bind.call("fsb_comm_broadcast_dma", *head, self.peers(off), t.data_ptr(), t.numel() * t.element_size(), owner,
                   _bind.status_ptr(self.device), _bind.stream_ptr(self.device), launches=2)

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
                         weights: Optional[torch.Tensor], rows_per_token: int, lane: int = 0,
                         fill: Optional[Tuple[torch.Tensor, int, int, int]] = None) -> None:
        """Store row ``t // rows_per_token`` of ``x`` into row ``dst_row[t]`` of rank ``dst_rank[t]``'s ``dst`` (heap tensor).
        ``fill = (counts[2E] int32, E, C, n_local)``: also zero the rows of this rank's segments that no token claimed
        (``dst`` laid out ``[n_local, world, C, M]``, expert ``e`` having taken ``counts[e] + counts[E + e]`` slots)."""
        ln = self._lane(lane)
        off = self.offset_of(dst)
        assert off is not None, "destination must live in the symmetric heap"
        _bind.call("fsb_comm_moe_scatter_rows", *self._head(ln), self._counter(ln), self.peers(off), x.data_ptr(), dst_rank.data_ptr(),
                   dst_row.data_ptr(), _bind.ptr(weights), dst_rank.numel(), rows_per_token, x.shape[-1],
                   None if fill is None else fill[0].data_ptr(), 0 if fill is None else fill[1], 0 if fill is None else fill[2],
                   0 if fill is None else fill[3], _bind.status_ptr(self.device), _bind.stream_ptr(self.device))

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


def set_timeout(seconds: float) -> None:
    """Limit of one device-side wait for a peer in every collective launched from now on (default 30 s, or
    ``FSB200_COMM_TIMEOUT_S``).  When a wait runs out the kernel records an error in the device status word and returns;
    the host raises :class:`fairscale_b200.utils.failure.CommTimeoutError` at its next status check."""
    _sigs()
    _bind.call("fsb_comm_set_timeout_ms", int(max(1, round(seconds * 1000))))


def stream_memops_available() -> bool:
    """True when the driver exports stream-ordered memory writes (needed by the copy-engine weight-gather GEMM)."""
    return bool(_bind.fn("fsb_comm_stream_memops_available")())


def timeout_ms() -> int:
    """The current limit of one device-side wait for a peer, in milliseconds."""
    fn = _bind.fn("fsb_comm_get_timeout_ms")
    fn.restype = ctypes.c_longlong
    return int(fn())


def available() -> bool:
    """True when the native library is present and torch exposes symmetric memory on this build."""
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return _native.available() and torch.cuda.is_available() and torch.cuda.device_count() > 1
