"""Sequence-parallel tensor-parallel linears whose collective runs inside the GEMM kernel.

``all_gather_linear(x_shard, W, b, group)``      : ``y = all_gather(x_shard) @ W^T + b``            (column-parallel)
``linear_reduce_scatter(x, W, b, group)``        : ``y_shard = reduce_scatter(x @ W^T) + b``        (row-parallel)

With an NVLink workspace for ``group`` (:func:`fairscale_b200.parallel.nvlink.enable`) and bf16 CUDA tensors each
call is ONE kernel of ``csrc/gemm_comm_tcgen05.cu``: copy / reduce CTAs move chunks over peer memory while the
tcgen05 CTAs compute the chunks in an order that hides the transfer.  The backward of each is the other fused
kernel (the gradient of an all-gather is a reduce-scatter and vice versa) plus a local wgrad GEMM on the
already-gathered operand, so a transformer layer does no stand-alone tensor-parallel collective at all.  The
reference does these steps as ``all_reduce`` + ``F.linear`` (fairscale/nn/model_parallel/layers.py:290,380-382;
mappings.py:42-78).

Anywhere else (CPU, gloo, other dtypes, shapes the kernels do not take) the same functions run the collective
and the matmul separately through :mod:`fairscale_b200.parallel.comm`.
"""

from __future__ import annotations

import os
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..ops import _bind
from ..ops import gemm as gemm_ops
from ..ops.reduce import column_sum
from . import comm, nvlink, symm

_AG_CHANNEL, _RS_CHANNEL, _WAG_CHANNEL, _WAG_DMA_CHANNEL, _AG_DMA_CHANNEL = 16, 18, 20, 22, 24  # signal-pad channels (entry / flags, exit) outside the collective lanes
_SIGS_DONE = False


def _sigs() -> None:
    global _SIGS_DONE
    if _SIGS_DONE:
        return
    from ctypes import c_int, c_uint, c_void_p

    head = [c_int, c_int, c_uint, c_int, c_void_p, c_void_p]
    S = _bind._SIGNATURES
    S["fsb_ag_gemm_bf16"] = head + [c_void_p] * 7 + [c_int] * 7 + [c_void_p, c_uint, c_int, c_void_p, c_void_p]
    S["fsb_gemm_rs_bf16"] = head + [c_void_p] * 6 + [c_int] * 6 + [c_void_p, c_uint, c_uint, c_int, c_void_p, c_void_p]
    S["fsb_gemm_rs_arrivals"] = [c_int, c_int, c_int]
    from ctypes import c_longlong

    S["fsb_wag_gemm_bf16"] = head + [c_void_p, c_longlong, c_void_p, c_longlong] + [c_void_p] * 4 + [c_int] * 6 + [c_void_p, c_uint, c_int,
                                                                                                                     c_void_p, c_void_p]
    _SIGS_DONE = True


def comm_ctas(remote_bytes: float = 0.0, flops: float = 0.0, world: int = 2) -> int:
    """CTAs (SMs) of a fused kernel that move data instead of computing.

    Enough of them to move ``remote_bytes`` over NVLink while the remaining SMs spend ``flops`` on the chunks that do
    not depend on the transfer; one copy CTA (bulk copies, 192 KB in flight) sustains roughly 60 GB/s of peer reads.  ``FSB200_FUSED_COMM_CTAS`` overrides."""
    env = os.environ.get("FSB200_FUSED_COMM_CTAS")
    if env:
        return int(env)
    if remote_bytes <= 0 or flops <= 0:
        return 16
    overlap_s = flops / 1.2e15 * max(world - 1, 1) / world
    need = remote_bytes / max(overlap_s, 1e-6) / 60e9
    return int(min(24, max(6, -(-need // 1))))


class _State:
    """Per-workspace bookkeeping of the fused kernels: epochs, monotonic chunk counters and their targets."""

    def __init__(self, ws: Any):
        self.ws = ws
        dev = ws.device
        self.ag_counts = torch.zeros(16, dtype=torch.int32, device=dev)
        self.rs_counts = torch.zeros(16, dtype=torch.int32, device=dev)
        self.ag_target = 0
        self.rs_target = 0
        self.rs_target_comm = 0
        self.ag_epoch = 0
        self.rs_epoch = 0
        self.wag_counts = torch.zeros(16, dtype=torch.int32, device=dev)
        self.wag_target = 0
        self.wag_epoch = 0
        self.wag_flags = torch.zeros(256, dtype=torch.int32, device=dev)  # piece arrivals of the copy-engine variant
        self.wag_flag_epoch = 0
        self.wag_stream: Optional[torch.cuda.Stream] = None
        self.acc: Dict[int, torch.Tensor] = {}


_STATES: Dict[int, _State] = {}


def _state(ws: Any) -> _State:
    st = _STATES.get(id(ws))
    if st is None:
        _sigs()
        st = _STATES[id(ws)] = _State(ws)
    return st


def _workspace(group: Any, *tensors: torch.Tensor) -> Optional[Any]:
    if comm.comm_mode() == "nccl" or not all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors):
        return None
    if not _bind.use_native(*tensors):
        return None
    return symm.workspace_for(group if group is not None else dist.group.WORLD)


def ag_gemm_supported(ws: Any, Mc: int, K: int, N: int) -> bool:
    return ws is not None and Mc % 128 == 0 and K % 8 == 0 and N % 8 == 0


def gemm_rs_supported(ws: Any, M: int, K: int, N: int) -> bool:
    return ws is not None and M % ws.world == 0 and (M // ws.world) % 128 == 0 and K % 8 == 0 and N % 8 == 0


# ---------------------------------------------------------------------------------------------- raw kernels
AG_PIECE_BYTES = 4 << 20  # granularity of the arrival flags of the copy-engine all-gather -> GEMM


def ag_gemm_engine() -> str:
    """``"sm"`` (default): copy CTAs inside the GEMM launch; ``"dma"``: copy engines gather the activation blocks while the
    CTA-pair GEMM, visiting its tiles in arrival order, waits on per-piece flags.  ``FSB200_AG_GEMM_ENGINE`` selects.
    Measured at 2 GPUs (16384 x 6144 x 4096): sm 641 us, dma 737 us, NCCL all-gather + GEMM 724 us - the dma variant pays for
    copying the rank's own block into the gathered buffer in front of the GEMM, which the copy CTAs hide."""
    return os.environ.get("FSB200_AG_GEMM_ENGINE", "sm")


def ag_gemm(ws: Any, x_shard: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], *, w_is_kn: bool = False,
            gelu: bool = False, engine: Optional[str] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(y[M, N], gathered[M, K])`` with ``M = world * Mc``.  ``w`` is ``[N, K]``, or ``[K, N]`` when ``w_is_kn``."""
    st = _state(ws)
    Mc, K = x_shard.shape
    N = w.shape[1] if w_is_kn else w.shape[0]
    M = Mc * ws.world
    dev = x_shard.device
    window = ws.scratch("ag_in", (Mc, K), torch.bfloat16)
    if ws.offset_of(x_shard) is None or not x_shard.is_contiguous():
        window.copy_(x_shard)
        src_off = ws.offset_of(window)
        block = window
    else:
        src_off = ws.offset_of(x_shard)
        block = x_shard
    gathered = torch.empty((M, K), dtype=torch.bfloat16, device=dev)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    engine = engine or ag_gemm_engine()
    piece_rows = max(128, AG_PIECE_BYTES // (2 * K) // 128 * 128)
    pieces = ws.world * -(-Mc // piece_rows)
    if engine == "dma" and M >= 256 and N >= 256 and pieces <= st.wag_flags.numel() and nvlink.stream_memops_available():
        # Same structure as the copy-engine weight gather: barriers and the own block on the GEMM's stream, only peer
        # copies (copy engines) and driver-side flag stores beside the GEMM.
        cur = torch.cuda.current_stream(dev)
        if st.wag_stream is None:
            st.wag_stream = torch.cuda.Stream(device=dev)
        side = st.wag_stream
        st.wag_flag_epoch = (st.wag_flag_epoch + 1) & 0x3FFFFFFF
        ws.barrier_on(_AG_DMA_CHANNEL, 2 * st.wag_flag_epoch)  # every peer's block is final
        piece_bytes = piece_rows * K * 2
        ws.gather_blocks_flagged(gathered, block, piece_bytes, st.wag_flags, st.wag_flag_epoch, phase=0)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            ws.gather_blocks_flagged(gathered, block, piece_bytes, st.wag_flags, st.wag_flag_epoch, phase=1)
        _bind.call("fsb_gemm_bf16_streamed_a", gathered.data_ptr(), w.data_ptr(), y.data_ptr(), _bind.ptr(bias), M, N, K, w.stride(0), N,
                   int(w_is_kn), 0 if bias is None else (2 if gelu else 1), st.wag_flags.data_ptr(), st.wag_flag_epoch, Mc, piece_rows,
                   ws.rank, ws.world, nvlink.timeout_ms(), _bind.status_ptr(dev), _bind.stream_ptr(dev))
        cur.wait_stream(side)
        ws.barrier_on(_AG_DMA_CHANNEL, 2 * st.wag_flag_epoch + 1)  # every peer is done reading this rank's block
        for t in (gathered, block, st.wag_flags):
            t.record_stream(side)
        return y, gathered
    n_comm = comm_ctas((ws.world - 1) * Mc * K * 2.0, 2.0 * M * N * K, ws.world)
    st.ag_epoch = (st.ag_epoch + 1) & 0x7FFFFFFF
    st.ag_target = (st.ag_target + n_comm) & 0xFFFFFFFF
    epi = 0 if bias is None else (2 if gelu else 1)
    a_local = ws.base + src_off
    _bind.call(
        "fsb_ag_gemm_bf16", ws.rank, ws.world, st.ag_epoch, _AG_CHANNEL, ws.pad_ptrs, ws.counters.data_ptr() + 4 * 16,
        ws.peers(src_off), a_local, gathered.data_ptr(), w.data_ptr(), y.data_ptr(), _bind.ptr(bias), None,
        M, N, K, w.stride(0), N, int(w_is_kn), epi, st.ag_counts.data_ptr(), st.ag_target, n_comm,
        _bind.status_ptr(dev), _bind.stream_ptr(dev),
    )
    return y, gathered


def weight_gather_gemm_supported(ws: Any, shard: torch.Tensor, full: torch.Tensor, w_offset: int, N: int, K: int) -> bool:
    """The fused all-gather + first GEMM of an FSDP unit needs: the shard in the symmetric heap, bf16, 16-byte friendly
    sizes and offsets, the weight rows inside the gathered buffer and at most 64 N tiles."""
    return (ws is not None and shard.dtype == torch.bfloat16 and full.dtype == torch.bfloat16 and ws.offset_of(shard) is not None
            and shard.is_contiguous() and full.is_contiguous() and full.numel() == shard.numel() * ws.world
            and (shard.numel() * 2) % 16 == 0 and shard.data_ptr() % 16 == 0 and full.data_ptr() % 16 == 0
            and w_offset % 8 == 0 and K % 8 == 0 and w_offset + N * K <= full.numel() and (N + 255) // 256 <= 64)


WAG_PIECE_BYTES = 4 << 20  # granularity of the arrival flags of the copy-engine variant


def weight_gather_engine() -> str:
    """``"dma"`` (default): copy engines move the shards while the CTA-pair GEMM waits on per-piece arrival flags;
    ``"sm"``: copy CTAs inside the GEMM's own launch pull the shards.  ``FSB200_WAG_ENGINE`` selects."""
    return os.environ.get("FSB200_WAG_ENGINE", "dma")


def weight_gather_gemm(ws: Any, x: torch.Tensor, shard: torch.Tensor, full: torch.Tensor, w_offset: int, N: int, K: int,
                       bias: Optional[torch.Tensor] = None, *, gelu: bool = False, n_comm: Optional[int] = None,
                       engine: Optional[str] = None) -> torch.Tensor:
    """``y[M, N] = x[M, K] @ W^T (+ bias)`` where ``W = full[w_offset : w_offset + N * K].view(N, K)`` and ``full`` - the
    gathered flat parameter of an FSDP unit - is filled from every rank's ``shard`` (heap resident) while the product
    runs.  On return (in stream order) ``full`` is complete.  ``bias`` must already hold valid data.

    Engine ``"dma"``: behind a flag barrier on the current stream, the copy engines of a side stream move the shards,
    weight rows first, and the driver stores a flag per 4 MB piece; the GEMM on the current stream visits its tiles in
    row order of W and waits for the pieces under each tile; a second barrier follows the GEMM.  Engine ``"sm"``: one
    launch whose copy CTAs pull the shards and whose GEMM CTAs wait on their chunk counters."""
    st = _state(ws)
    x = x.contiguous()
    M = x.shape[0]
    dev = x.device
    y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    engine = engine or weight_gather_engine()
    if (engine == "dma" and not gelu and M >= 256 and N >= 256 and -(-N * K * 2 // WAG_PIECE_BYTES) <= st.wag_flags.numel()
            and nvlink.stream_memops_available()):
        # Only copies from peers (copy engines) and driver-side flag stores run beside the GEMM.  Both barriers and the
        # copy of this rank's own rows of W are enqueued on the GEMM's stream, before / after it: nothing the GEMM waits
        # for depends on finding room on an SM next to it.
        cur = torch.cuda.current_stream(dev)
        if st.wag_stream is None:
            st.wag_stream = torch.cuda.Stream(device=dev)
        side = st.wag_stream
        st.wag_flag_epoch = (st.wag_flag_epoch + 1) & 0x3FFFFFFF
        ws.barrier_on(_WAG_DMA_CHANNEL, 2 * st.wag_flag_epoch)  # every peer's shard is final
        rng = (w_offset, w_offset + N * K)
        # every rank starts at a different piece of W: the weight sits in the shards of a few ranks, which all the others
        # would otherwise read at the same moment
        first = (ws.rank * -(-N * K * 2 // WAG_PIECE_BYTES)) // ws.world
        ws.gather_flagged_copies(full, shard, rng, WAG_PIECE_BYTES, st.wag_flags, st.wag_flag_epoch, phase=0)  # own rows of W
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            ws.gather_flagged_copies(full, shard, rng, WAG_PIECE_BYTES, st.wag_flags, st.wag_flag_epoch, phase=1, first_piece=first)
        _bind.call("fsb_gemm_bf16_streamed_b", x.data_ptr(), full.data_ptr() + 2 * w_offset, y.data_ptr(), _bind.ptr(bias), M, N, K,
                   x.stride(0), N, 0 if bias is None else 1, st.wag_flags.data_ptr(), st.wag_flag_epoch, WAG_PIECE_BYTES, first,
                   nvlink.timeout_ms(), _bind.status_ptr(dev), _bind.stream_ptr(dev))
        cur.wait_stream(side)  # the rest of the flat parameter
        ws.barrier_on(_WAG_DMA_CHANNEL, 2 * st.wag_flag_epoch + 1)  # every peer is done reading this rank's shard
        for t in (full, shard, st.wag_flags):
            t.record_stream(side)
        return y
    remote = (ws.world - 1) * shard.numel() * 2.0
    n_comm = n_comm if n_comm is not None else comm_ctas(remote, 2.0 * M * N * K, ws.world)
    st.wag_epoch = (st.wag_epoch + 1) & 0x7FFFFFFF
    st.wag_target = (st.wag_target + n_comm) & 0xFFFFFFFF
    epi = 0 if bias is None else (2 if gelu else 1)
    _bind.call(
        "fsb_wag_gemm_bf16", ws.rank, ws.world, st.wag_epoch, _WAG_CHANNEL, ws.pad_ptrs, ws.counters.data_ptr() + 4 * 20,
        ws.peers(ws.offset_of(shard)), shard.numel(), full.data_ptr(), w_offset, x.data_ptr(), y.data_ptr(), _bind.ptr(bias), None,
        M, N, K, x.stride(0), N, epi, st.wag_counts.data_ptr(), st.wag_target, n_comm, _bind.status_ptr(dev), _bind.stream_ptr(dev),
    )
    return y


def gemm_rs(ws: Any, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], *, w_is_kn: bool = False) -> torch.Tensor:
    """``out[Mc, N] = (sum over ranks of x @ w^T)[this rank's rows] + bias``; ``x`` is ``[M, K_local]``."""
    st = _state(ws)
    M, K = x.shape
    N = w.shape[1] if w_is_kn else w.shape[0]
    Mc = M // ws.world
    dev = x.device
    x = x.contiguous()
    stage = ws.scratch("rs_stage", (M, N), torch.bfloat16)
    recv_elems = max(ws.world - 1, 1) * Mc * N  # one bf16 receive buffer per peer
    acc = st.acc.get(recv_elems)
    if acc is None:
        acc = st.acc[recv_elems] = torch.empty(recv_elems, dtype=torch.bfloat16, device=dev)
    out = torch.empty((Mc, N), dtype=torch.bfloat16, device=dev)
    n_comm = comm_ctas((ws.world - 1) * Mc * N * 2.0, 2.0 * M * N * K, ws.world)
    arrivals = _bind.fn("fsb_gemm_rs_arrivals")(M, N, ws.world)
    st.rs_epoch = (st.rs_epoch + 1) & 0x7FFFFFFF
    st.rs_target = (st.rs_target + arrivals) & 0xFFFFFFFF
    if ws.world > 1:
        st.rs_target_comm = (st.rs_target_comm + n_comm) & 0xFFFFFFFF
    _bind.call(
        "fsb_gemm_rs_bf16", ws.rank, ws.world, st.rs_epoch, _RS_CHANNEL, ws.pad_ptrs, ws.counters.data_ptr() + 4 * 17,
        ws.peers(ws.offset_of(stage)), x.data_ptr(), w.data_ptr(), out.data_ptr(), _bind.ptr(bias), acc.data_ptr(),
        M, N, K, x.stride(0), w.stride(0), int(w_is_kn), st.rs_counts.data_ptr(), st.rs_target, st.rs_target_comm, n_comm,
        _bind.status_ptr(dev), _bind.stream_ptr(dev),
    )
    return out


# ---------------------------------------------------------------------------------------------- unfused path
def _all_gather_rows(x: torch.Tensor, group: Any) -> torch.Tensor:
    world = comm.group_size(group)
    out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    comm.all_gather_into(out.view(-1), x.contiguous().view(-1), group=group)
    return out


def _reduce_scatter_rows(x: torch.Tensor, group: Any) -> torch.Tensor:
    world = comm.group_size(group)
    out = torch.empty((x.shape[0] // world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if world > 1 and dist.get_backend(group) == "gloo":  # gloo has no reduce-scatter
        full = x.contiguous().clone()
        dist.all_reduce(full, group=group)
        r = comm.group_rank(group)
        out.copy_(full[r * out.shape[0] : (r + 1) * out.shape[0]])
        return out
    comm.reduce_scatter_into(out.view(-1), x.contiguous().view(-1), group=group)
    return out


def _plain_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The local product of the unfused routes: the library's own tcgen05 GEMM for bf16 on the GPU (no autograd here, the
    callers are autograd functions), ``F.linear`` for everything else (CPU, other dtypes)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
        return gemm_ops.linear_forward(x, w, bias)[0]
    return F.linear(x, w, bias)


# ---------------------------------------------------------------------------------------------- autograd
class _AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], group: Any) -> torch.Tensor:  # type: ignore[override]
        ctx.group = group
        ws = _workspace(group, x, w)
        if ag_gemm_supported(ws, x.shape[0], x.shape[1], w.shape[0]):
            y, gathered = ag_gemm(ws, x, w, bias)
            ctx.fused = True
        else:
            gathered = _all_gather_rows(x, group)
            y = _plain_linear(gathered, w, bias)
            ctx.fused = False
        ctx.save_for_backward(gathered, w)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx: Any, dy: torch.Tensor) -> Any:  # type: ignore[override]
        gathered, w = ctx.saved_tensors
        dy = dy.contiguous()
        ws = _workspace(ctx.group, dy, w) if ctx.fused else None
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            if gemm_rs_supported(ws, dy.shape[0], dy.shape[1], w.shape[1]):
                dx = gemm_rs(ws, dy, w, None, w_is_kn=True)  # dX = reduce_scatter(dY @ W)
            else:
                dx = _reduce_scatter_rows(dy @ w, ctx.group)
        if ctx.needs_input_grad[1]:
            dw = gemm_ops.linear_wgrad(dy, gathered).to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = column_sum(dy) if _bind.use_native(dy) and dy.dtype == torch.bfloat16 else dy.sum(0)
        return dx, dw, db, None


class _LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], group: Any) -> torch.Tensor:  # type: ignore[override]
        ctx.group = group
        ws = _workspace(group, x, w)
        if gemm_rs_supported(ws, x.shape[0], x.shape[1], w.shape[0]):
            out = gemm_rs(ws, x, w, bias)
            ctx.fused = True
        else:
            out = _reduce_scatter_rows(_plain_linear(x, w), group)
            if bias is not None:
                out = out + bias
            ctx.fused = False
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return out

    @staticmethod
    def backward(ctx: Any, dout: torch.Tensor) -> Any:  # type: ignore[override]
        x, w = ctx.saved_tensors
        dout = dout.contiguous()
        ws = _workspace(ctx.group, dout, w) if ctx.fused else None
        dx = dw = db = None
        if ag_gemm_supported(ws, dout.shape[0], dout.shape[1], w.shape[1]):
            dx, gathered = ag_gemm(ws, dout, w, None, w_is_kn=True)  # dX = all_gather(dOut) @ W
        else:
            gathered = _all_gather_rows(dout, ctx.group)
            dx = gathered @ w if ctx.needs_input_grad[0] else None
        if ctx.needs_input_grad[1]:
            dw = gemm_ops.linear_wgrad(gathered, x).to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            # the bias is replicated but every rank saw different tokens: sum its gradient over the group
            db = (column_sum(dout) if _bind.use_native(dout) and dout.dtype == torch.bfloat16 else dout.sum(0)).clone()
            if comm.group_size(ctx.group) > 1:
                comm.all_reduce(db, group=ctx.group)
        return dx, dw, db, None


def _flatten(x: torch.Tensor) -> Tuple[torch.Tensor, Tuple[int, ...]]:
    return x.reshape(-1, x.shape[-1]), tuple(x.shape[:-1])


def all_gather_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], group: Any = None) -> torch.Tensor:
    """``x``: this rank's token shard ``[tokens / world, ..., K]`` (sharded along dim 0); returns ``[tokens, ..., N_local]``."""
    x2, lead = _flatten(x)
    y = _AllGatherLinear.apply(x2, weight, bias, group)
    world = comm.group_size(group)
    return y.view((lead[0] * world,) + lead[1:] + (y.shape[-1],)) if lead else y


def linear_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], group: Any = None) -> torch.Tensor:
    """``x``: ``[tokens, ..., K_local]``; returns this rank's token shard ``[tokens / world, ..., N]`` of the reduced product."""
    x2, lead = _flatten(x)
    y = _LinearReduceScatter.apply(x2, weight, bias, group)
    world = comm.group_size(group)
    return y.view((lead[0] // world,) + lead[1:] + (y.shape[-1],)) if lead else y


class _LinearAllReduce(torch.autograd.Function):
    """``y = all_reduce(x @ w^T) + bias`` with the whole result on every rank: the API-exact output of a row-parallel
    linear (fairscale/nn/model_parallel/layers.py:380-386).  With a workspace the reduction is the fused
    GEMM -> reduce-scatter kernel followed by an NVLink all-gather of the reduced rows (an all-reduce is a reduce-scatter
    plus an all-gather anyway; here the first half overlaps the tensor-core work).  Backward is the ``g`` operator's:
    the incoming gradient is already whole on every rank, so ``dX = dY W`` and ``dW = dY^T X`` are local products."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], group: Any) -> torch.Tensor:  # type: ignore[override]
        ws = _workspace(group, x, w)
        world = comm.group_size(group)
        if world > 1 and x.shape[0] % world == 0 and gemm_rs_supported(ws, x.shape[0], x.shape[1], w.shape[0]):
            y = _all_gather_rows(gemm_rs(ws, x, w, bias), group)
        else:
            y = _plain_linear(x, w)
            if world > 1:
                comm.all_reduce(y, group=group)
            if bias is not None:
                y = y + bias
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx: Any, dy: torch.Tensor) -> Any:  # type: ignore[override]
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm_ops.linear_dgrad(dy, w) if ctx.needs_input_grad[0] else None  # tcgen05 GEMM on the GPU, matmul elsewhere
        dw = gemm_ops.linear_wgrad(dy, x).to(w.dtype) if ctx.needs_input_grad[1] else None
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = column_sum(dy) if _bind.use_native(dy) and dy.dtype == torch.bfloat16 else dy.sum(0)
        return dx, dw, db, None


def linear_all_reduce(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], group: Any = None) -> torch.Tensor:
    """``x``: ``[tokens, ..., K_local]``; returns the fully reduced ``[tokens, ..., N]`` on every rank (the bias is added
    once, after the reduction)."""
    x2, lead = _flatten(x)
    y = _LinearAllReduce.apply(x2, weight, bias, group)
    return y.view(lead + (y.shape[-1],)) if lead else y
