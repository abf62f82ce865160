"""LayerNorm / RMSNorm (``csrc/norm.cu``): bf16 in/out, fp32 statistics, fused affine."""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from . import _bind


def _native_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    H = x.shape[-1]
    return _bind.use_native(x, w) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and H % 8 == 0 and H <= 8192


def norm_forward(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, rms: bool
                 ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    H = x.shape[-1]
    if not _native_ok(x, weight):
        xf = x.float()
        if rms:
            rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
            y = xf * rstd * weight.float()
            mean = None
        else:
            mean = xf.mean(-1, keepdim=True)
            rstd = torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + eps)
            y = (xf - mean) * rstd * weight.float()
            if bias is not None:
                y = y + bias.float()
        return y.to(x.dtype), mean, rstd
    x2 = x.contiguous().view(-1, H)
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    mean = None if rms else torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _bind.call("fsb_norm_fwd", x2.data_ptr(), weight.data_ptr(), _bind.ptr(bias), y.data_ptr(), _bind.ptr(mean), rstd.data_ptr(),
               rows, H, eps, int(rms), _bind.stream_ptr(x.device))
    return y.view_as(x), mean, rstd


def norm_backward(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, mean: Optional[torch.Tensor], rstd: torch.Tensor,
                  rms: bool, has_bias: bool) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    H = x.shape[-1]
    if not _native_ok(x, weight):
        xf, dyf, wf = x.float(), dy.float(), weight.float()
        xhat = xf * rstd if rms else (xf - mean) * rstd
        wdy = dyf * wf
        c2 = (wdy * xhat).mean(-1, keepdim=True)
        c1 = 0 if rms else wdy.mean(-1, keepdim=True)
        dx = (wdy - c1 - xhat * c2) * rstd
        dw = (dyf * xhat).reshape(-1, H).sum(0)
        db = dyf.reshape(-1, H).sum(0) if has_bias else None
        return dx.to(x.dtype), dw.to(weight.dtype), None if db is None else db.to(weight.dtype)
    x2, dy2 = x.contiguous().view(-1, H), dy.contiguous().view(-1, H)
    rows = x2.shape[0]
    strips = _bind.fn("fsb_norm_bwd_num_strips")(rows)
    partials = torch.empty((2, strips, H), dtype=torch.float32, device=x.device)
    dx = torch.empty_like(x2)
    dw = torch.empty(H, dtype=torch.bfloat16, device=x.device)
    db = torch.empty(H, dtype=torch.bfloat16, device=x.device) if (has_bias and not rms) else None
    _bind.call("fsb_norm_bwd", dy2.data_ptr(), x2.data_ptr(), weight.data_ptr(), _bind.ptr(mean), rstd.data_ptr(), dx.data_ptr(),
               dw.data_ptr(), _bind.ptr(db), partials.data_ptr(), rows, H, int(rms), _bind.stream_ptr(x.device),
               launches=4 if db is not None else 3)
    return dx.view_as(x), dw, db


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps: float, rms: bool):  # type: ignore[override]
        y, mean, rstd = norm_forward(x, weight, bias, eps, rms)
        ctx.rms = rms
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x, weight, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, weight, mean, rstd = ctx.saved_tensors
        dx, dw, db = norm_backward(dy, x, weight, mean, rstd, ctx.rms, ctx.has_bias)
        return dx, dw, db, None, None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float = 1e-5) -> torch.Tensor:
    return _NormFn.apply(x, weight, bias, eps, False)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return _NormFn.apply(x, weight, None, eps, True)


class LayerNorm(nn.Module):
    """Drop-in ``nn.LayerNorm`` over the last dimension running the fused kernel on CUDA bf16 inputs."""

    def __init__(self, hidden: int, eps: float = 1e-5, bias: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden))
        self.bias = nn.Parameter(torch.zeros(hidden)) if bias else None
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return layer_norm(x, self.weight, self.bias, self.eps)


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return rms_norm(x, self.weight, self.eps)
