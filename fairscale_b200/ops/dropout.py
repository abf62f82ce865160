"""Dropout whose mask is regenerated, not stored (``csrc/misc.cu``: ``fsb_dropout``).

The mask of element ``e`` is word ``e % 4`` of Philox4x32-10 at counter ``offset + e // 4`` under the key ``seed``.
``seed`` and ``offset`` come from the device's default CUDA generator and the offset is advanced past the counters
used, so ``torch.cuda.get_rng_state`` / ``set_rng_state`` (activation checkpointing, the model-parallel RNG tracker)
reproduce the mask on recomputation.  Replaces ``nn.Dropout`` of the reference's benchmark model
(benchmarks/models/transformer_lm.py:38,55,57 in the reference).
"""

from __future__ import annotations

from typing import Any, Tuple

import torch

from . import _bind


def _take_counters(device: torch.device, n: int) -> Tuple[int, int]:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    gen = torch.cuda.default_generators[idx]
    seed, offset = gen.initial_seed(), gen.get_offset()
    gen.set_offset(offset + ((n + 3) // 4 + 3) // 4 * 4)  # generator offsets move in multiples of 4
    return seed, offset


def dropout_apply(x: torch.Tensor, p: float, seed: int, offset: int) -> torch.Tensor:
    """``x`` times the keep mask of ``(seed, offset)`` times ``1 / (1 - p)`` (bf16 CUDA tensors)."""
    x = x.contiguous()
    y = torch.empty_like(x)
    _bind.call("fsb_dropout", x.data_ptr(), y.data_ptr(), x.numel(), float(p), seed & (2**64 - 1), offset, _bind.stream_ptr(x.device))
    return y


class _DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, p: float) -> torch.Tensor:  # type: ignore[override]
        ctx.p = p
        ctx.seed, ctx.offset = _take_counters(x.device, x.numel())
        return dropout_apply(x, p, ctx.seed, ctx.offset)

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> Any:  # type: ignore[override]
        return dropout_apply(g, ctx.p, ctx.seed, ctx.offset), None


def dropout(x: torch.Tensor, p: float = 0.1, training: bool = True) -> torch.Tensor:
    if not training or p == 0.0:
        return x
    if not _bind.use_native(x) or x.dtype != torch.bfloat16:
        return torch.nn.functional.dropout(x, p, training)
    return _DropoutFn.apply(x, p)


class Dropout(torch.nn.Module):
    """Drop-in for ``nn.Dropout`` that stores no mask on CUDA bf16 inputs."""

    def __init__(self, p: float = 0.1) -> None:
        super().__init__()
        if p < 0.0 or p >= 1.0:
            raise ValueError(f"dropout probability has to be in [0, 1), got {p}")
        self.p = p

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return dropout(x, self.p, self.training)

    def extra_repr(self) -> str:
        return f"p={self.p}"
