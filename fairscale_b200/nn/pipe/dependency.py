"""Ordering edges for autograd: ``fork`` splits a zero-size token off a tensor, ``join`` ties a token to another tensor.

After ``a, token = fork(a)`` and ``b = join(b, token)`` the backward of everything that produced ``b`` runs before the
backward of what produced ``a`` continues, because ``a``'s producer now also waits for the token's (empty) gradient.
The pipeline uses this to replay micro-batches in reverse order on every stage and to place recomputation right before
the backward it serves.  Same contract as fairscale/nn/pipe/dependency.py:29-67.
"""

from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch
from torch import Tensor

from .phony import get_phony

__all__: List[str] = []


def _tracked(*tensors: Tensor) -> bool:
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


class Fork(torch.autograd.Function):
    """(x) -> (x, token).  The token's gradient is ignored; what matters is that this node has two consumers."""

    @staticmethod
    def forward(ctx: Any, x: Tensor) -> Tuple[Tensor, Tensor]:  # type: ignore[override]
        ctx.set_materialize_grads(False)  # an unused token contributes None, not a zero tensor
        token = get_phony(x.device, requires_grad=False)
        return x.detach(), token.detach()

    @staticmethod
    def backward(ctx: Any, grad_x: Optional[Tensor], grad_token: Optional[Tensor]) -> Optional[Tensor]:  # type: ignore[override]
        return grad_x


class Join(torch.autograd.Function):
    """(x, token) -> x.  The token gets no gradient, but its producer is now upstream of x's consumers."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, token: Tensor) -> Tensor:  # type: ignore[override]
        return x.detach()

    @staticmethod
    def backward(ctx: Any, grad_x: Tensor) -> Tuple[Tensor, None]:  # type: ignore[override]
        return grad_x, None


def fork(input: Tensor) -> Tuple[Tensor, Tensor]:
    if _tracked(input):
        return Fork.apply(input)
    return input, get_phony(input.device, requires_grad=False)


def join(input: Tensor, phony: Tensor) -> Tensor:
    return Join.apply(input, phony) if _tracked(input, phony) else input
