"""Column reductions (bias gradients) on ``csrc/norm.cu``'s strip-partial kernels."""

from __future__ import annotations

import torch

from . import _bind


def column_sum(x: torch.Tensor) -> torch.Tensor:
    """``x.sum(0)`` for a 2-D bf16 matrix, accumulated in fp32 without atomics."""
    x2 = x.reshape(-1, x.shape[-1])
    rows, H = x2.shape
    if not _bind.use_native(x2) or x2.dtype != torch.bfloat16 or H % 8:
        return x2.float().sum(0).to(x.dtype)
    x2 = x2.contiguous()
    strips = _bind.fn("fsb_colsum_num_strips")(rows)
    partials = torch.empty((strips, H), dtype=torch.float32, device=x.device)
    out = torch.empty((H,), dtype=torch.bfloat16, device=x.device)
    _bind.call("fsb_colsum", x2.data_ptr(), rows, H, partials.data_ptr(), out.data_ptr(), _bind.stream_ptr(x.device), launches=2)
    return out
