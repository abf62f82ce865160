"""Causal multi-head self-attention.

``causal_attention(qkv, n_heads)`` takes the packed projection ``[B, S, 3*H*D]`` and returns ``[B, S, H*D]``.
CUDA bf16 inputs run the hand-written kernels of ``csrc/attention.cu`` when they are present in the
native library; otherwise (and on CPU) a PyTorch formulation is used and :data:`BACKEND` says so.
"""

from __future__ import annotations

import math
import warnings
from typing import Optional

import torch

from . import _bind

BACKEND = "unset"
_WARNED_LIBRARY_PATH = False  # the fall-back to the library kernel is announced once


def _reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """fp32 attention oracle on [B, H, S, D] tensors."""
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    n = s.shape[-1]
    s = s.masked_fill(torch.ones(n, n, dtype=torch.bool, device=s.device).triu(1), float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), v.float())


def _native_available() -> bool:
    from .. import _native

    try:
        return hasattr(_native.lib(), "fsb_attn_fwd")
    except Exception:
        return False


def causal_attention(qkv: torch.Tensor, n_heads: int, scale: Optional[float] = None) -> torch.Tensor:
    global BACKEND
    B, S, three_hd = qkv.shape
    D = three_hd // (3 * n_heads)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _bind.use_native(qkv) and qkv.dtype == torch.bfloat16 and _native_available() and D in (64, 128) and S % 128 == 0:
        from .attention_native import flash_attention_packed

        BACKEND = "tcgen05"
        return flash_attention_packed(qkv, n_heads, scale)
    q, k, v = qkv.view(B, S, 3, n_heads, D).permute(2, 0, 3, 1, 4)
    if qkv.is_cuda:
        global _WARNED_LIBRARY_PATH
        if not _WARNED_LIBRARY_PATH:
            _WARNED_LIBRARY_PATH = True
            warnings.warn(
                f"causal_attention: the tcgen05 kernels take bf16 with head size 64 or 128 and a sequence length that is a multiple "
                f"of 128 (got {qkv.dtype}, head size {D}, length {S}); this call runs torch's scaled_dot_product_attention instead",
                stacklevel=2,
            )
        BACKEND = "torch-sdpa"
        o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale)
    else:
        BACKEND = "reference"
        o = _reference(q, k, v, scale).to(qkv.dtype)
    return o.transpose(1, 2).reshape(B, S, n_heads * D)
