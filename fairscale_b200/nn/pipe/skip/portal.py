"""Portals carry skip tensors around the autograd graph (parity: fairscale/nn/pipe/skip/portal.py:42-272).

A skip tensor that crosses partitions must not be captured by the checkpoint of the partitions in between.
The portal keeps the tensor outside the graph and threads three tiny autograd nodes through phony tensors:
``blue`` (where it is stashed; returns the gradient there), ``copy`` (device move at the stage boundary) and
``orange`` (where it is popped; collects the gradient).  ``tensor_life`` counts how many more times the tensor
will be requested (forward, recomputation) so it is released exactly when no longer needed.
"""

from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch
from torch import Tensor

from ..copy import Context as CopyContext
from ..copy import Copy
from ..phony import get_phony
from ..stream import AbstractStream, get_device
from .namespace import Namespace

__all__: List[str] = []


class Portal:
    def __init__(self, tensor: Optional[Tensor], tensor_life: int, index: int = 0) -> None:
        self.put_tensor(tensor, tensor_life)
        self.grad: Optional[Tensor] = None
        self.__index = index
        self.ns_name: Optional[Tuple[Namespace, str]] = None

    @property
    def index(self) -> int:
        return self.__index

    def blue(self) -> Tensor:
        tensor = self.use_tensor()
        if tensor is None:
            return get_phony(torch.device("cpu"), requires_grad=False)
        return PortalBlue.apply(self, tensor)

    def orange(self, phony: Tensor) -> Optional[Tensor]:
        self.check_tensor_life()
        if self.tensor is None:
            return self.use_tensor()
        return PortalOrange.apply(self, phony)

    def copy(self, prev_stream: AbstractStream, next_stream: AbstractStream, phony: Tensor) -> Tensor:
        if self.tensor is None:
            return get_phony(torch.device("cpu"), requires_grad=False)
        return PortalCopy.apply(self, prev_stream, next_stream, phony)

    def check_tensor_life(self) -> None:
        if self.tensor_life <= 0:
            raise RuntimeError("tensor in portal has been removed")

    def put_tensor(self, tensor: Optional[Tensor], tensor_life: int) -> None:
        self.tensor_life = tensor_life
        self.tensor = tensor if tensor_life > 0 else None

    def use_tensor(self) -> Optional[Tensor]:
        self.check_tensor_life()
        tensor = self.tensor
        self.tensor_life -= 1
        if self.tensor_life <= 0:
            self.tensor = None
        return tensor

    def put_grad(self, grad: Tensor) -> None:
        self.grad = grad

    def use_grad(self) -> Tensor:
        if self.grad is None:
            raise RuntimeError("grad in portal has been removed or never set")
        grad, self.grad = self.grad, None
        return grad


class Context(CopyContext):
    portal: Portal


class PortalBlue(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, portal: Portal, tensor: Tensor) -> Tensor:  # type: ignore[override]
        ctx.portal = portal
        return get_phony(tensor.device, requires_grad=False).detach()

    @staticmethod
    def backward(ctx: Any, grad_phony: Tensor) -> Tuple[None, Tensor]:  # type: ignore[override]
        return None, ctx.portal.use_grad()


class PortalOrange(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, portal: Portal, phony: Tensor) -> Tensor:  # type: ignore[override]
        ctx.portal = portal
        tensor = portal.use_tensor()
        assert tensor is not None
        return tensor.detach()

    @staticmethod
    def backward(ctx: Any, grad: Tensor) -> Tuple[None, None]:  # type: ignore[override]
        ctx.portal.put_grad(grad)
        return None, None


class PortalCopy(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, portal: Portal, prev_stream: AbstractStream, next_stream: AbstractStream, phony: Tensor) -> Tensor:  # type: ignore[override]
        ctx.portal = portal
        assert portal.tensor is not None
        (portal.tensor,) = Copy.forward(ctx, prev_stream, next_stream, portal.tensor)
        return get_phony(get_device(next_stream), requires_grad=False).detach()

    @staticmethod
    def backward(ctx: Any, grad_phony: Tensor) -> Tuple[None, None, None, None]:  # type: ignore[override]
        portal = ctx.portal
        assert portal.grad is not None
        _, _, portal.grad = Copy.backward(ctx, portal.grad)
        return None, None, None, None
