"""BatchNorm whose running statistics follow the mini-batch, not the micro-batch.

Parity: fairscale/nn/pipe/batchnorm.py:37-172.  Each micro-batch is normalised with its own batch statistics
(as GPipe requires), while sums and squared sums are accumulated across the ``chunks`` micro-batches and folded
into ``running_mean`` / ``running_var`` once per mini-batch; recomputation passes are not counted.
"""

from __future__ import annotations

from typing import Optional, TypeVar, cast

import torch
import torch.nn.functional as F
from torch import Tensor, nn
from torch.nn.modules.batchnorm import _BatchNorm

from .checkpoint import is_recomputing

__all__ = ["DeferredBatchNorm"]

TModule = TypeVar("TModule", bound=nn.Module)


class DeferredBatchNorm(_BatchNorm):
    sum: Tensor
    sum_squares: Tensor

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: Optional[float] = 0.1, affine: bool = True, chunks: int = 1) -> None:
        super().__init__(num_features, eps, momentum, affine, track_running_stats=True)
        self.register_buffer("sum", torch.zeros_like(self.running_mean))
        self.register_buffer("sum_squares", torch.zeros_like(self.running_var))
        self.counter = 0
        self.tracked = 0
        self.chunks = chunks

    def _check_input_dim(self, input: Tensor) -> None:
        if input.dim() <= 2:
            raise ValueError("expected at least 3D input (got %dD input)" % input.dim())

    def _track(self, input: Tensor) -> bool:
        """Accumulate this micro-batch; True once all ``chunks`` micro-batches were seen."""
        reduce_dims = [0] + list(range(2, input.dim()))
        with torch.no_grad():
            self.sum += input.sum(reduce_dims)
            self.sum_squares += (input**2).sum(reduce_dims)
        self.counter += input.numel() // input.size(1)
        self.tracked += 1
        return self.tracked == self.chunks

    def _commit(self) -> None:
        """Fold the accumulated mini-batch statistics into the running ones."""
        self.num_batches_tracked += 1
        factor = 1.0 / float(self.num_batches_tracked) if self.momentum is None else self.momentum
        mean = self.sum / self.counter
        var = self.sum_squares / self.counter - mean**2
        self.running_mean.mul_(1 - factor).add_(mean * factor)
        self.running_var.mul_(1 - factor).add_(var * factor)
        self.sum.zero_()
        self.sum_squares.zero_()
        self.counter = 0
        self.tracked = 0

    def forward(self, input: Tensor) -> Tensor:  # type: ignore[override]
        if not self.training:
            return F.batch_norm(input, self.running_mean, self.running_var, self.weight, self.bias, False, 0.0, self.eps)
        if not is_recomputing():
            if self._track(input):
                self._commit()
        return F.batch_norm(input, None, None, self.weight, self.bias, True, 0.0, self.eps)

    @classmethod
    def convert_deferred_batch_norm(cls, module: TModule, chunks: int = 1) -> TModule:
        """Recursively replace tracking BatchNorm layers by deferred ones sharing the same parameters and buffers."""
        if isinstance(module, DeferredBatchNorm) and module.chunks is chunks:
            return cast(TModule, module)
        out: nn.Module = module
        if isinstance(module, _BatchNorm) and module.track_running_stats:
            out = DeferredBatchNorm(module.num_features, module.eps, module.momentum, module.affine, chunks)
            if module.affine:
                out.register_parameter("weight", module.weight)
                out.register_parameter("bias", module.bias)
            out.register_buffer("running_mean", module.running_mean)
            out.register_buffer("running_var", module.running_var)
            out.register_buffer("num_batches_tracked", module.num_batches_tracked)
        for name, child in module.named_children():
            out.add_module(name, cls.convert_deferred_batch_norm(child, chunks))
        return cast(TModule, out)
