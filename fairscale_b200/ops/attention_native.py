"""autograd wrapper of the tcgen05 flash-attention kernels (``csrc/attention.cu``) for packed QKV."""

from __future__ import annotations

import torch

from . import _bind

_BOUND = False


def _bind_sigs() -> None:
    global _BOUND
    if _BOUND:
        return
    from ctypes import c_float, c_int, c_void_p

    _bind._SIGNATURES["fsb_attn_fwd"] = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
    _bind._SIGNATURES["fsb_attn_bwd"] = [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p]
    _BOUND = True


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv: torch.Tensor, n_heads: int, scale: float):  # type: ignore[override]
        _bind_sigs()
        B, S, three_hd = qkv.shape
        D = three_hd // (3 * n_heads)
        qkv = qkv.contiguous()
        o = torch.empty((B, S, n_heads * D), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((B, n_heads, S), dtype=torch.float32, device=qkv.device)
        _bind.call("fsb_attn_fwd", qkv.data_ptr(), o.data_ptr(), lse.data_ptr(), B, S, n_heads, D, scale,
                   _bind.status_ptr(qkv.device), _bind.stream_ptr(qkv.device))
        ctx.save_for_backward(qkv, o, lse)
        ctx.n_heads, ctx.scale = n_heads, scale
        return o

    @staticmethod
    def backward(ctx, d_o: torch.Tensor):  # type: ignore[override]
        qkv, o, lse = ctx.saved_tensors
        B, S, three_hd = qkv.shape
        H = ctx.n_heads
        D = three_hd // (3 * H)
        d_o = d_o.contiguous()
        dqkv = torch.empty_like(qkv)
        delta = torch.empty((2,) + tuple(lse.shape), dtype=torch.float32, device=lse.device)  # scale*delta, then base-2 lse
        _bind.call("fsb_attn_bwd", qkv.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(), delta.data_ptr(), dqkv.data_ptr(),
                   B, S, H, D, ctx.scale, _bind.status_ptr(qkv.device), _bind.stream_ptr(qkv.device), launches=3)
        return dqkv, None, None


def flash_attention_packed(qkv: torch.Tensor, n_heads: int, scale: float) -> torch.Tensor:
    """Causal attention on packed ``qkv [B, S, 3*H*D]`` (bf16, S % 128 == 0, D in {64, 128}) -> ``[B, S, H*D]``."""
    return _FlashAttnFn.apply(qkv, n_heads, scale)
