"""Rotary position embedding on packed QKV (``csrc/misc.cu``: ``fsb_rope``)."""

from __future__ import annotations

from typing import Any

import torch

from . import _bind


def rope_reference(qkv: torch.Tensor, theta: float, backward: bool = False, pos_offset: int = 0) -> torch.Tensor:
    """fp32 PyTorch statement of the kernel: rotate the interleaved pairs of q and k of ``[B, S, 3, H, D]``."""
    B, S, _, H, Dh = qkv.shape
    pos = torch.arange(pos_offset, pos_offset + S, device=qkv.device, dtype=torch.float32)
    inv = theta ** (-torch.arange(0, Dh, 2, device=qkv.device, dtype=torch.float32) / Dh)
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, :, None, None, :], ang.sin()[None, :, None, None, :]
    if backward:
        sin = -sin
    qk = qkv[:, :, :2].float()
    x1, x2 = qk[..., 0::2], qk[..., 1::2]
    rot = torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).flatten(-2)
    return torch.cat([rot.to(qkv.dtype), qkv[:, :, 2:]], dim=2)


def _rope_apply(qkv: torch.Tensor, theta: float, backward: bool, pos_offset: int) -> torch.Tensor:
    B, S, three, H, D = qkv.shape
    assert three == 3
    if not _bind.use_native(qkv) or qkv.dtype != torch.bfloat16 or D % 8:
        return rope_reference(qkv, theta, backward, pos_offset)
    qkv = qkv.contiguous()
    out = torch.empty_like(qkv)
    _bind.call("fsb_rope", qkv.data_ptr(), out.data_ptr(), B, S, H, D, float(theta), int(backward), int(pos_offset),
               _bind.stream_ptr(qkv.device))
    return out


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, qkv: torch.Tensor, theta: float, pos_offset: int) -> torch.Tensor:  # type: ignore[override]
        ctx.theta, ctx.pos_offset = theta, pos_offset
        return _rope_apply(qkv, theta, False, pos_offset)

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> Any:  # type: ignore[override]
        # a rotation's Jacobian is orthogonal: the gradient is rotated back by the same angle
        return _rope_apply(g, ctx.theta, True, ctx.pos_offset), None, None


def rope_qkv(qkv: torch.Tensor, theta: float = 10000.0, pos_offset: int = 0) -> torch.Tensor:
    """Apply rotary embeddings to the q and k parts of packed ``[B, S, 3, H, D]``; v passes through."""
    return _RopeFn.apply(qkv, theta, pos_offset)
