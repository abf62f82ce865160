"""Dtype conversion with 16-byte accesses (``csrc/elementwise.cu``): master shard -> compute shard, gradient
shard -> master precision.  Replaces the ATen copies at
fairscale/nn/data_parallel/fully_sharded_data_parallel.py:2257-2266 and :1752-1756."""

from __future__ import annotations

from typing import Optional

import torch

from . import _bind


def cast_into(dst: torch.Tensor, src: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``dst.copy_(src * scale)`` across fp32 / fp16 / bf16."""
    if (
        _bind.use_native(dst, src)
        and dst.is_contiguous()
        and src.is_contiguous()
        and dst.numel() == src.numel()
        and dst.device == src.device
        and src.dtype in _bind._DTYPE_CODE
        and dst.dtype in _bind._DTYPE_CODE
        and (src.dtype == torch.float32 or dst.dtype == torch.float32 or src.dtype == dst.dtype)
    ):
        _bind.call("fsb_cast", src.data_ptr(), _bind.dtype_code(src.dtype), dst.data_ptr(), _bind.dtype_code(dst.dtype),
                   src.numel(), scale, _bind.stream_ptr(src.device))
        return dst
    if scale != 1.0:
        dst.copy_(src.to(torch.float32) * scale)
    else:
        dst.copy_(src, non_blocking=True)
    return dst


def cast(src: torch.Tensor, dtype: torch.dtype, scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty_like(src, dtype=dtype)
    return cast_into(out, src, scale)
