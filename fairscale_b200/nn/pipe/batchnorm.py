"""BatchNorm whose running statistics see the whole mini-batch although the layer only ever sees micro-batches.

Normalisation itself uses each micro-batch's own statistics (as ``nn.BatchNorm`` in training mode does); the *running*
mean and variance are updated once per mini-batch from sums accumulated over its ``chunks`` micro-batches, so they
match what an un-piped model would have tracked.  Contract of fairscale/nn/pipe/batchnorm.py:34-172.
"""

from __future__ import annotations

from typing import Optional, TypeVar, cast

import torch
from torch import Tensor, nn
import torch.nn.functional as F
from torch.nn.modules.batchnorm import _BatchNorm

from .checkpoint import is_recomputing

__all__ = ["DeferredBatchNorm"]

TModule = TypeVar("TModule", bound=nn.Module)


class DeferredBatchNorm(_BatchNorm):
    sum: Tensor
    sum_squares: Tensor

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: Optional[float] = 0.1, affine: bool = True, chunks: int = 1) -> None:
        super().__init__(num_features, eps, momentum, affine, track_running_stats=True)
        for name in ("sum", "sum_squares"):  # per-channel totals of the current mini-batch (part of the state dict)
            self.register_buffer(name, torch.zeros(num_features))
        self.chunks = chunks
        self.counter = 0  # elements per channel behind the totals
        self.tracked = 0  # micro-batches behind the totals

    def _check_input_dim(self, input: Tensor) -> None:
        if input.dim() < 3:
            raise ValueError("expected at least 3D input (got %dD input)" % input.dim())

    @torch.no_grad()
    def _accumulate(self, x: Tensor) -> None:
        """Add one micro-batch to the totals."""
        per_channel = x.transpose(0, 1).reshape(x.size(1), -1)
        self.sum.add_(per_channel.sum(1))
        self.sum_squares.add_(per_channel.square().sum(1))
        self.counter += per_channel.size(1)
        self.tracked += 1

    @torch.no_grad()
    def _fold_into_running_stats(self) -> None:
        """The mini-batch is complete: update the running statistics from the totals and clear them."""
        self.num_batches_tracked += 1
        # momentum None means a cumulative average over all mini-batches seen so far
        step = self.momentum if self.momentum is not None else 1.0 / float(self.num_batches_tracked)
        batch_mean = self.sum / self.counter
        batch_var = self.sum_squares / self.counter - batch_mean.square()
        self.running_mean.mul_(1 - step).add_(batch_mean, alpha=step)
        self.running_var.mul_(1 - step).add_(batch_var, alpha=step)
        self.sum.zero_()
        self.sum_squares.zero_()
        self.counter = self.tracked = 0

    def forward(self, input: Tensor) -> Tensor:  # type: ignore[override]
        use_batch_stats = self.training
        if use_batch_stats and not is_recomputing():  # a recomputed forward must not count its micro-batch twice
            self._accumulate(input)
            if self.tracked == self.chunks:
                self._fold_into_running_stats()
        mean, var = (None, None) if use_batch_stats else (self.running_mean, self.running_var)
        return F.batch_norm(input, mean, var, self.weight, self.bias, use_batch_stats, 0.0, self.eps)

    @classmethod
    def convert_deferred_batch_norm(cls, module: TModule, chunks: int = 1) -> TModule:
        """``module`` with every ``_BatchNorm`` that tracks running statistics replaced by a deferred one (weights,
        statistics and counters carried over); other modules are converted in place, child by child."""
        already = isinstance(module, DeferredBatchNorm) and module.chunks == chunks
        if already or not isinstance(module, _BatchNorm):
            if not already:
                for name, child in list(module.named_children()):
                    setattr(module, name, cls.convert_deferred_batch_norm(child, chunks))
            return module
        if not module.track_running_stats:
            return module
        twin = cls(module.num_features, module.eps, module.momentum, module.affine, chunks)
        carried = ["running_mean", "running_var", "num_batches_tracked"] + (["weight", "bias"] if module.affine else [])
        for name in carried:
            setattr(twin, name, getattr(module, name))  # parameters and buffers are shared, not copied
        return cast(TModule, twin)
