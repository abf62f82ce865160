"""bf16 matrix products on the tcgen05 kernel (``csrc/gemm_tcgen05.cu``) and the autograd linear built on it.

Storage convention: every operand is a row-major 2-D bf16 tensor.  ``gemm(a, b, trans_a, trans_b)``
computes ``op(a) @ op(b)^T``-style products without materialising transposes by telling the kernel
which operand dimension is contiguous:

* ``linear_forward``  ``y[M,N] = x[M,K] @ w[N,K]^T``      (A K-major, B K-major)
* ``linear_dgrad``    ``dx[M,K] = dy[M,N] @ w[N,K]``      (A K-major, B MN-major)
* ``linear_wgrad``    ``dw[N,K] = dy[M,N]^T @ x[M,K]``    (A MN-major, B MN-major)

On CPU tensors (unit tests without a GPU) the same functions run a PyTorch reference.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _bind

EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL, EPI_DGELU, EPI_RESIDUAL = range(6)


class PendingGather:
    """A flat parameter whose all-gather has been deferred to the first product that reads one of its matrices
    (registered by FullyShardedDataParallel for units that opt in).  ``full`` is the gathered buffer (the parameter
    views point into it), ``shard`` this rank's heap-resident slice; small parameters are already in place."""

    def __init__(self, workspace, shard: torch.Tensor, full: torch.Tensor, stream=None) -> None:  # type: ignore[no-untyped-def]
        self.workspace, self.shard, self.full = workspace, shard, full
        self.stream = stream  # the stream that owns the workspace's all-gather lane (None: a private one)
        self.lo = full.data_ptr()
        self.hi = self.lo + full.numel() * full.element_size()

    def owns(self, t: torch.Tensor) -> bool:
        return self.lo <= t.data_ptr() < self.hi

    def finish_unfused(self) -> None:
        """Complete the gather with the ordinary collective (the consumer cannot use the fused kernel)."""
        if self.stream is None:
            self.workspace.all_gather(self.full, self.shard)
            return
        cur = torch.cuda.current_stream(self.full.device)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            self.workspace.all_gather(self.full, self.shard)
        cur.wait_stream(self.stream)


_PENDING_GATHERS: list = []


def defer_gather(pending: PendingGather) -> PendingGather:
    _PENDING_GATHERS.append(pending)
    return pending


def complete_deferred_gather(pending: PendingGather) -> None:
    """Gather now if ``pending`` is still waiting (its unit finished without a product that could take the fused route)."""
    for i, pg in enumerate(_PENDING_GATHERS):
        if pg is pending:
            _PENDING_GATHERS.pop(i).finish_unfused()
            return


def _take_pending(w: torch.Tensor) -> Optional[PendingGather]:
    for i, pg in enumerate(_PENDING_GATHERS):
        if pg.owns(w):
            return _PENDING_GATHERS.pop(i)
    return None


def _as_2d(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.is_contiguous() else t2.contiguous()


def _launch(
    a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, M: int, N: int, K: int, a_mn: bool, b_mn: bool, epilogue: int = EPI_NONE,
    bias: Optional[torch.Tensor] = None, aux: Optional[torch.Tensor] = None, aux_out: Optional[torch.Tensor] = None,
    accumulate: bool = False, max_ctas: int = 0,
) -> None:
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "tcgen05 GEMM takes bf16 operands"
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and c.stride(-1) == 1
    ld_aux = 0
    if aux is not None:
        ld_aux = aux.stride(0)
    elif aux_out is not None:
        ld_aux = aux_out.stride(0)
    _bind.call(
        "fsb_gemm_bf16",
        a.data_ptr(), b.data_ptr(), c.data_ptr(), _bind.ptr(bias), _bind.ptr(aux), _bind.ptr(aux_out),
        M, N, K, a.stride(0), b.stride(0), c.stride(0), ld_aux, int(a_mn), int(b_mn), epilogue,
        int(c.dtype == torch.float32), int(accumulate), max_ctas, _bind.status_ptr(a.device), _bind.stream_ptr(a.device),
    )


def linear_forward(
    x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *, gelu: bool = False,
    residual: Optional[torch.Tensor] = None, save_pre_activation: bool = False, out_dtype: Optional[torch.dtype] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``y = act(x @ w^T + bias) (+ residual)``; returns ``(y, pre_activation or None)``.

    ``x``: [..., K] bf16, ``w``: [N, K] bf16.  With ``gelu`` and ``save_pre_activation`` the kernel
    also writes ``x @ w^T + bias`` (needed by the backward) in the same pass.
    """
    x2 = _as_2d(x)
    M, K = x2.shape
    N = w.shape[0]
    out_dtype = out_dtype or torch.bfloat16
    if not _bind.use_native(x2, w):
        pre = torch.nn.functional.linear(x2.float(), w.float(), None if bias is None else bias.float())
        y = torch.nn.functional.gelu(pre) if gelu else pre
        if residual is not None:
            y = y + _as_2d(residual).float()
        pre_out = pre.to(x.dtype) if (gelu and save_pre_activation) else None
        return y.to(out_dtype if x.dtype == torch.bfloat16 else x.dtype).view(*x.shape[:-1], N), pre_out
    if _PENDING_GATHERS:
        pending = _take_pending(w)
        if pending is not None:
            from ..parallel import fused_tp

            w_offset = (w.data_ptr() - pending.lo) // 2
            plain = not gelu and residual is None and out_dtype == torch.bfloat16 and w.is_contiguous()
            if plain and fused_tp.weight_gather_gemm_supported(pending.workspace, pending.shard, pending.full, w_offset, N, K):
                # the unit's parameter all-gather runs inside this product's kernel
                y = fused_tp.weight_gather_gemm(pending.workspace, x2, pending.shard, pending.full, w_offset, N, K, bias)
                return y.view(*x.shape[:-1], N), None
            pending.finish_unfused()
    y = torch.empty((M, N), dtype=out_dtype, device=x.device)
    pre_out = None
    w = w if w.is_contiguous() else w.contiguous()
    if gelu:
        assert bias is not None and residual is None
        if save_pre_activation:
            pre_out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        _launch(x2, w, y, M, N, K, False, False, EPI_BIAS_GELU, bias=bias, aux_out=pre_out)
    elif residual is not None:
        r2 = _as_2d(residual)
        _launch(x2, w, y, M, N, K, False, False, EPI_BIAS_RESIDUAL if bias is not None else EPI_RESIDUAL, bias=bias, aux=r2)
    else:
        _launch(x2, w, y, M, N, K, False, False, EPI_BIAS if bias is not None else EPI_NONE, bias=bias)
    return y.view(*x.shape[:-1], N), pre_out


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, *, dgelu_pre: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dx = dy @ w`` (optionally multiplied by ``gelu'(dgelu_pre)`` in the epilogue).  ``dy``: [M, N], ``w``: [N, K]."""
    dy2 = _as_2d(dy)
    M, N = dy2.shape
    K = w.shape[1]
    if not _bind.use_native(dy2, w):
        dx = dy2.float() @ w.float()
        if dgelu_pre is not None:
            p = _as_2d(dgelu_pre).float()
            cdf = 0.5 * (1 + torch.erf(p * 0.7071067811865476))
            pdf = torch.exp(-0.5 * p * p) * 0.3989422804014327
            dx = dx * (cdf + p * pdf)
        return dx.to(dy.dtype)
    dx = torch.empty((M, K), dtype=torch.bfloat16, device=dy.device)
    w = w if w.is_contiguous() else w.contiguous()
    # output dim of this product is K (rows of the MN-major operand w[N, K]); reduction runs over N
    if dgelu_pre is not None:
        _launch(dy2, w, dx, M, K, N, False, True, EPI_DGELU, aux=_as_2d(dgelu_pre))
    else:
        _launch(dy2, w, dx, M, K, N, False, True)
    return dx


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, *, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """``dw[N, K] = dy[M, N]^T @ x[M, K]``.  ``out`` may be an fp32 buffer to accumulate into (``accumulate=True``)."""
    dy2, x2 = _as_2d(dy), _as_2d(x)
    M, N = dy2.shape
    K = x2.shape[1]
    if not _bind.use_native(dy2, x2):
        dw = dy2.float().t() @ x2.float()
        if out is not None:
            out.copy_(out + dw if accumulate else dw)
            return out
        return dw.to(dy.dtype)
    if out is None:
        out = torch.empty((N, K), dtype=torch.bfloat16, device=dy.device)
    _launch(dy2, x2, out, N, K, M, True, True, accumulate=accumulate)
    return out


def grad_slot_info(weight: torch.Tensor):
    """Forward-time capture of a weight's flat-gradient window descriptor (None for ordinary tensors)."""
    return getattr(weight, "_fsb_grad_slot", None)


def wgrad_into_slot(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, slot_info=None) -> torch.Tensor:
    """``dw`` for ``weight``; written straight into the flat-gradient window of ``weight`` when it has one."""
    slot = None
    info = slot_info if slot_info is not None else getattr(weight, "_fsb_grad_slot", None)
    if info is not None and dy.is_cuda and weight.dtype == torch.bfloat16:
        arena, offset, shape = info
        if (offset * 2) % 16 == 0:
            slot = arena.slot(offset, shape, weight.dtype, weight.device)
    return linear_wgrad(dy, x, out=slot)


def matmul_nt(a: torch.Tensor, b: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``a[M,K] @ b[N,K]^T`` for 2-D bf16 tensors."""
    y, _ = linear_forward(a, b, None, out_dtype=out_dtype)
    return y


class _LinearFn(torch.autograd.Function):
    """``y = x w^T + b`` with optional fused GELU or residual; backward uses the dgrad / wgrad products."""

    @staticmethod
    def forward(ctx, x, w, bias, gelu: bool, residual):  # type: ignore[override]
        need_grad = any(ctx.needs_input_grad)  # all False under no_grad
        y, pre = linear_forward(x, w, bias, gelu=gelu, residual=residual, save_pre_activation=gelu and need_grad)
        ctx.gelu = gelu
        ctx.has_bias = bias is not None
        ctx.has_residual = residual is not None
        ctx.w_slot = grad_slot_info(w)
        ctx.save_for_backward(x, w, pre)
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, w, pre = ctx.saved_tensors
        dy2 = _as_2d(dy)
        d_res = dy if ctx.has_residual else None
        if ctx.gelu:
            from .activations import gelu_backward

            dy2 = gelu_backward(dy2, pre)
        dx = linear_dgrad(dy2, w).view_as(x) if ctx.needs_input_grad[0] else None
        dw = wgrad_into_slot(dy2, x, w, ctx.w_slot) if ctx.needs_input_grad[1] else None
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from .reduce import column_sum

            db = column_sum(dy2)
        return dx, dw, db, None, d_res


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *, gelu: bool = False,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable fused linear: ``gelu(x w^T + b)`` or ``x w^T + b + residual``."""
    return _LinearFn.apply(x, w, bias, gelu, residual)


# ---------------------------------------------------------------------------------------------- grouped (batched) products
def _launch_batched(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, M: int, N: int, K: int, a_mn: bool, b_mn: bool,
                    epilogue: int = EPI_NONE, bias: Optional[torch.Tensor] = None, aux: Optional[torch.Tensor] = None,
                    aux_out: Optional[torch.Tensor] = None) -> None:
    """``c[e] = epilogue(a[e] * b[e]^T)`` for 3-D contiguous-last-dim tensors with a common leading (expert) dimension."""
    from ctypes import c_int, c_longlong, c_void_p

    _bind._SIGNATURES.setdefault("fsb_gemm_bf16_batched", [c_void_p] * 6 + [c_int] * 8 + [c_longlong] * 5 + [c_int] * 5 + [c_void_p, c_void_p])
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 3 and b.dim() == 3 and c.dim() == 3
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and c.stride(-1) == 1
    ref = aux if aux is not None else aux_out
    _bind.call(
        "fsb_gemm_bf16_batched", a.data_ptr(), b.data_ptr(), c.data_ptr(), _bind.ptr(bias), _bind.ptr(aux), _bind.ptr(aux_out),
        a.shape[0], M, N, K, a.stride(1), b.stride(1), c.stride(1), 0 if ref is None else ref.stride(1),
        a.stride(0), b.stride(0), c.stride(0), 0 if ref is None else ref.stride(0), 0 if bias is None else bias.stride(0),
        int(a_mn), int(b_mn), epilogue, int(c.dtype == torch.float32), 0, _bind.status_ptr(a.device), _bind.stream_ptr(a.device),
    )


def _batched_native(*ts: torch.Tensor) -> bool:
    return _bind.use_native(*ts) and all(t.dtype == torch.bfloat16 for t in ts)


def batched_linear_forward(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *, gelu: bool = False,
                           save_pre_activation: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``y[e] = act(x[e] @ w[e]^T + bias[e])`` for ``x [E, C, K]``, ``w [E, N, K]``, ``bias [E, N]``: one launch for all experts."""
    E, C, K = x.shape
    N = w.shape[1]
    if not _batched_native(x, w):
        pre = torch.baddbmm(bias.float().unsqueeze(1), x.float(), w.float().transpose(1, 2)) if bias is not None else torch.bmm(x.float(), w.float().transpose(1, 2))
        y = torch.nn.functional.gelu(pre) if gelu else pre
        return y.to(x.dtype), (pre.to(x.dtype) if gelu and save_pre_activation else None)
    x, w = x.contiguous(), w.contiguous()
    y = torch.empty((E, C, N), dtype=torch.bfloat16, device=x.device)
    pre = torch.empty_like(y) if (gelu and save_pre_activation) else None
    if gelu:
        assert bias is not None
        _launch_batched(x, w, y, C, N, K, False, False, EPI_BIAS_GELU, bias=bias.contiguous(), aux_out=pre)
    else:
        _launch_batched(x, w, y, C, N, K, False, False, EPI_BIAS if bias is not None else EPI_NONE, bias=None if bias is None else bias.contiguous())
    return y, pre


def batched_linear_dgrad(dy: torch.Tensor, w: torch.Tensor, *, dgelu_pre: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``dx[e] = dy[e] @ w[e]`` (times ``gelu'(pre[e])`` when given): ``dy [E, C, N]``, ``w [E, N, K]`` -> ``[E, C, K]``."""
    E, C, N = dy.shape
    K = w.shape[2]
    if not _batched_native(dy, w):
        dx = torch.bmm(dy.float(), w.float())
        if dgelu_pre is not None:
            p = dgelu_pre.float()
            dx = dx * (0.5 * (1 + torch.erf(p * 0.7071067811865476)) + p * torch.exp(-0.5 * p * p) * 0.3989422804014327)
        return dx.to(dy.dtype)
    dy, w = dy.contiguous(), w.contiguous()
    dx = torch.empty((E, C, K), dtype=torch.bfloat16, device=dy.device)
    if dgelu_pre is not None:
        _launch_batched(dy, w, dx, C, K, N, False, True, EPI_DGELU, aux=dgelu_pre.contiguous())
    else:
        _launch_batched(dy, w, dx, C, K, N, False, True)
    return dx


def batched_linear_wgrad(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``dw[e] = dy[e]^T @ x[e]``: ``dy [E, C, N]``, ``x [E, C, K]`` -> ``[E, N, K]``."""
    E, C, N = dy.shape
    K = x.shape[2]
    if not _batched_native(dy, x):
        return torch.bmm(dy.float().transpose(1, 2), x.float()).to(dy.dtype)
    dy, x = dy.contiguous(), x.contiguous()
    dw = torch.empty((E, N, K), dtype=torch.bfloat16, device=dy.device)
    _launch_batched(dy, x, dw, N, K, C, True, True)
    return dw


class _GroupedMLPFn(torch.autograd.Function):
    """``gelu(x w1^T + b1) w2^T + b2`` for every expert at once; four launches forward + recompute-free backward."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2):  # type: ignore[override]
        h, pre = batched_linear_forward(x, w1, b1, gelu=True, save_pre_activation=True)
        y, _ = batched_linear_forward(h, w2, b2)
        ctx.save_for_backward(x, w1, w2, pre, h)
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, w1, w2, pre, h = ctx.saved_tensors
        dy = dy.contiguous()
        dw2 = batched_linear_wgrad(dy, h)
        db2 = dy.float().sum(1).to(dy.dtype)
        dpre = batched_linear_dgrad(dy, w2, dgelu_pre=pre)
        dw1 = batched_linear_wgrad(dpre, x)
        db1 = dpre.float().sum(1).to(dy.dtype)
        dx = batched_linear_dgrad(dpre, w1)
        return dx, dw1, db1, dw2, db2


def grouped_mlp(x: torch.Tensor, w1: torch.Tensor, b1: torch.Tensor, w2: torch.Tensor, b2: torch.Tensor) -> torch.Tensor:
    """Feed-forward of ``E`` experts on ``x [E, C, M]``: ``w1 [E, F, M]``, ``b1 [E, F]``, ``w2 [E, M, F]``, ``b2 [E, M]``."""
    return _GroupedMLPFn.apply(x, w1, b1, w2, b2)
