"""Fused transformer feed-forward: ``y = gelu(x W1^T + b1) W2^T + b2 (+ residual)`` as one autograd node.

Four tensor-core launches forward+backward-critical fusions (all in ``csrc/gemm_tcgen05.cu`` epilogues):
bias+GELU (with the pre-activation written in the same pass when a backward will follow), bias+residual,
and GELU' applied to the first dgrad's output tile while it is still in registers.
"""

from __future__ import annotations

from typing import Optional

import torch

from .gemm import grad_slot_info, linear_dgrad, linear_forward, wgrad_into_slot
from .reduce import column_sum


class _MLPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):  # type: ignore[override]
        need_grad = any(ctx.needs_input_grad)  # all False under no_grad (e.g. the first pass of a checkpointed block)
        h, pre = linear_forward(x, w1, b1, gelu=True, save_pre_activation=need_grad)
        y, _ = linear_forward(h, w2, b2, residual=residual)
        ctx.has_residual = residual is not None
        ctx.slots = (grad_slot_info(w1), grad_slot_info(w2))
        ctx.save_for_backward(x, w1, w2, pre, h)
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, w1, w2, pre, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        d_pre = linear_dgrad(dy2, w2, dgelu_pre=pre)          # [M, ffn], already multiplied by gelu'(pre)
        dw2 = wgrad_into_slot(dy2, h, w2, ctx.slots[1])
        db2 = column_sum(dy2)
        dx = linear_dgrad(d_pre, w1).view_as(x)
        dw1 = wgrad_into_slot(d_pre, x, w1, ctx.slots[0])
        db1 = column_sum(d_pre)
        return dx, dw1, db1, dw2, db2, (dy if ctx.has_residual else None)


def mlp(x: torch.Tensor, w1: torch.Tensor, b1: torch.Tensor, w2: torch.Tensor, b2: torch.Tensor,
        residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _MLPFn.apply(x, w1, b1, w2, b2, residual)
