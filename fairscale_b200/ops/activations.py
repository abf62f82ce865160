"""GELU (erf form) and SwiGLU on bf16 tensors (``csrc/elementwise.cu``)."""

from __future__ import annotations

import torch

from . import _bind


def _gelu_grad_ref(x: torch.Tensor) -> torch.Tensor:
    cdf = 0.5 * (1 + torch.erf(x * 0.7071067811865476))
    pdf = torch.exp(-0.5 * x * x) * 0.3989422804014327
    return cdf + x * pdf


def gelu_forward(x: torch.Tensor) -> torch.Tensor:
    if not _bind.use_native(x) or x.dtype != torch.bfloat16 or x.numel() % 8:
        return torch.nn.functional.gelu(x.float()).to(x.dtype)
    x = x.contiguous()
    y = torch.empty_like(x)
    _bind.call("fsb_gelu", x.data_ptr(), None, y.data_ptr(), x.numel(), 0, _bind.stream_ptr(x.device))
    return y


def gelu_backward(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``dy * gelu'(x)``."""
    if not _bind.use_native(x, dy) or x.dtype != torch.bfloat16 or x.numel() % 8:
        return (dy.float() * _gelu_grad_ref(x.float())).to(dy.dtype)
    x, dy = x.contiguous(), dy.contiguous()
    dx = torch.empty_like(x)
    _bind.call("fsb_gelu", x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(), 1, _bind.stream_ptr(x.device))
    return dx


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):  # type: ignore[override]
        ctx.save_for_backward(x)
        return gelu_forward(x)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        (x,) = ctx.saved_tensors
        return gelu_backward(dy, x)


def gelu(x: torch.Tensor) -> torch.Tensor:
    return _GeluFn.apply(x)


def swiglu_forward(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dimension."""
    F = gate_up.shape[-1] // 2
    if not _bind.use_native(gate_up) or gate_up.dtype != torch.bfloat16 or F % 8:
        g, u = gate_up.float().split(F, dim=-1)
        return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)
    gu = gate_up.contiguous().view(-1, 2 * F)
    y = torch.empty((gu.shape[0], F), dtype=gate_up.dtype, device=gate_up.device)
    _bind.call("fsb_swiglu_fwd", gu.data_ptr(), y.data_ptr(), gu.shape[0], F, _bind.stream_ptr(gu.device))
    return y.view(*gate_up.shape[:-1], F)


def swiglu_backward(gate_up: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    F = gate_up.shape[-1] // 2
    if not _bind.use_native(gate_up, dy) or gate_up.dtype != torch.bfloat16 or F % 8:
        g, u = gate_up.float().split(F, dim=-1)
        d = dy.float()
        sig = torch.sigmoid(g)
        silu = g * sig
        return torch.cat([d * u * (sig + silu * (1 - sig)), d * silu], dim=-1).to(gate_up.dtype)
    gu = gate_up.contiguous().view(-1, 2 * F)
    d = dy.contiguous().view(-1, F)
    out = torch.empty_like(gu)
    _bind.call("fsb_swiglu_bwd", gu.data_ptr(), d.data_ptr(), out.data_ptr(), gu.shape[0], F, _bind.stream_ptr(gu.device))
    return out.view_as(gate_up)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):  # type: ignore[override]
        ctx.save_for_backward(gate_up)
        return swiglu_forward(gate_up)

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        (gate_up,) = ctx.saved_tensors
        return swiglu_backward(gate_up, dy)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    return _SwigluFn.apply(gate_up)


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """bf16 ``a + b`` in one pass (residual connections)."""
    if not _bind.use_native(a, b) or a.dtype != torch.bfloat16 or a.numel() % 8 or a.shape != b.shape:
        return a + b
    a, b = a.contiguous(), b.contiguous()
    y = torch.empty_like(a)
    _bind.call("fsb_add_bf16", a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), _bind.stream_ptr(a.device))
    return y


def softmax(x: torch.Tensor, scale: float = 1.0, causal: bool = False) -> torch.Tensor:
    """Row softmax over the last dimension with fp32 math; ``causal`` masks ``j > i`` of the last two dims."""
    if not _bind.use_native(x) or x.dtype not in (torch.float32, torch.bfloat16):
        xs = x.float() * scale
        if causal:
            n, m = x.shape[-2], x.shape[-1]
            mask = torch.ones(n, m, dtype=torch.bool, device=x.device).tril(diagonal=m - n)
            xs = xs.masked_fill(~mask, float("-inf"))
        return torch.softmax(xs, dim=-1).to(x.dtype)
    xc = x.contiguous()
    y = torch.empty_like(xc)
    cols = xc.shape[-1]
    rows = xc.numel() // cols
    causal_rows = xc.shape[-2] if causal else 0
    causal_off = cols - xc.shape[-2] if causal else 0
    _bind.call("fsb_softmax", xc.data_ptr(), y.data_ptr(), rows, cols, _bind.dtype_code(x.dtype), scale, causal_rows, causal_off,
               _bind.stream_ptr(x.device))
    return y
