"""Synchronised batch normalisation with one collective per pass.

Capability parity with fairscale/experimental/nn/sync_batchnorm.py:32-220 (statistics over the whole process
group, aware of activation checkpointing so the recomputation pass reuses the statistics of the first pass and
the running averages move once, ``convert_sync_batchnorm``).  The reference issues two all-reduces in forward
(count, then [mean, meansqr]); here forward all-reduces a single fp32 vector ``[sum, sumsq, count]`` and
backward a single ``[sum(dy), sum(dy * xhat)]``, which over NVLink is latency-bound, so halving the number of
collectives is what matters.  Statistics are accumulated in fp32 whatever the activation dtype.
"""

from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ...nn.checkpoint import checkpoint_invocations, is_checkpointing, is_recomputing


def _reduce_dims(x: Tensor) -> List[int]:
    return [d for d in range(x.ndim) if d != 1]


def _bshape(x: Tensor) -> List[int]:
    return [1, x.size(1)] + [1] * (x.ndim - 2)


def _calculate_stats(x: Tensor, eps: float, group: Any) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """(mean, var, invstd, total_count) over every rank of ``group``; fp32 vectors of length C (count: scalar)."""
    dims = _reduce_dims(x)
    xf = x.float()
    C = x.size(1)
    vec = torch.empty(2 * C + 1, dtype=torch.float32, device=x.device)
    vec[:C] = xf.sum(dims)
    vec[C : 2 * C] = (xf * xf).sum(dims)
    vec[2 * C] = x.numel() // C
    dist.all_reduce(vec, group=group)
    total = vec[2 * C]
    mean = vec[:C] / total
    var = (vec[C : 2 * C] / total - mean * mean).clamp_(min=0)
    return mean, var, torch.rsqrt(var + eps), total


class _SyncBatchNormFunction(torch.autograd.Function):
    """Normalise with given statistics; backward differentiates through the (global) statistics as well."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], mean: Tensor, invstd: Tensor,  # type: ignore[override]
                total: Tensor, group: Any) -> Tensor:
        ctx.save_for_backward(x, weight, mean, invstd, total)
        ctx.group = group
        shape = _bshape(x)
        scale = invstd if weight is None else invstd * weight.float()
        shift = -mean * scale if bias is None else bias.float() - mean * scale
        return torch.addcmul(shift.view(shape).to(x.dtype), x, scale.view(shape).to(x.dtype))

    @staticmethod
    def backward(ctx: Any, dy: Tensor) -> Any:  # type: ignore[override]
        x, weight, mean, invstd, total = ctx.saved_tensors
        dims, shape = _reduce_dims(x), _bshape(x)
        C = x.size(1)
        dyf = dy.float()
        xhat = (x.float() - mean.view(shape)) * invstd.view(shape)
        vec = torch.empty(2 * C, dtype=torch.float32, device=x.device)
        vec[:C] = dyf.sum(dims)
        vec[C:] = (dyf * xhat).sum(dims)
        grad_bias = vec[:C].clone() if ctx.needs_input_grad[2] else None
        grad_weight = vec[C:].clone() if ctx.needs_input_grad[1] else None
        grad_input = None
        if ctx.needs_input_grad[0]:
            dist.all_reduce(vec, group=ctx.group)
            g = invstd if weight is None else invstd * weight.float()
            mean_dy = (vec[:C] / total).view(shape)
            mean_dy_xhat = (vec[C:] / total).view(shape)
            grad_input = ((dyf - mean_dy - xhat * mean_dy_xhat) * g.view(shape)).to(x.dtype)
        if grad_weight is not None:
            grad_weight = grad_weight.to(weight.dtype)
        if grad_bias is not None:
            grad_bias = grad_bias.to(weight.dtype if weight is not None else dy.dtype)
        return grad_input, grad_weight, grad_bias, None, None, None, None


class SyncBatchNorm(torch.nn.BatchNorm2d):
    """Drop-in for ``torch.nn.SyncBatchNorm`` over ``process_group`` (default: WORLD); any ``[N, C, *]`` input."""

    def __init__(self, *args: Any, process_group: Any = None, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self._process_group = process_group
        self.saved_for_2nd_fwd: List[Tuple[Tensor, Tensor, Tensor]] = []
        # the statistics handed from the checkpointed pass to the recomputation make the BN patch unnecessary
        self.disable_patch_batchnorm = True

    def _check_input_dim(self, input: Tensor) -> None:
        if input.dim() < 2:
            raise ValueError(f"expected at least 2D input (got {input.dim()}D input)")

    def forward(self, input: Tensor) -> Tensor:  # type: ignore[override]
        self._check_input_dim(input)
        if not dist.is_initialized() or not self.training:
            return super().forward(input)
        group = self._process_group if self._process_group is not None else dist.group.WORLD
        # Statistics of a checkpointed call are handed to the repetition of that same call: they are kept in the call's own
        # scratch (one layer may run several times inside one call, and a step may have several calls that autograd
        # repeats in reverse order), or in this module's list when the checkpoint in use has no scratch.
        running = checkpoint_invocations()
        key = ("sync_batchnorm", id(self))
        stats = None
        if is_recomputing():
            for scratch in reversed(running):
                if scratch.get("_mode") == "replay" and scratch.get(key):
                    stats = scratch[key].pop(0)
                    break
            if stats is None and not running and self.saved_for_2nd_fwd:
                stats = self.saved_for_2nd_fwd.pop(0)
        if stats is None:
            with torch.no_grad():
                mean, var, invstd, total = _calculate_stats(input, self.eps, group)
                if self.track_running_stats and not is_recomputing():
                    m = self.momentum if self.momentum is not None else 1.0 / float(self.num_batches_tracked + 1)
                    self.running_mean += m * (mean.to(self.running_mean.dtype) - self.running_mean)
                    self.running_var += m * ((var * (total / (total - 1))).to(self.running_var.dtype) - self.running_var)
                    self.num_batches_tracked += 1
            stats = (mean, invstd, total)
        if running and running[-1].get("_mode") == "first":
            running[-1].setdefault(key, []).append(stats)  # the innermost call is in its forward: its repetition will ask
        elif not running and is_checkpointing() and not is_recomputing():
            self.saved_for_2nd_fwd.append(stats)
        mean, invstd, total = stats
        w = self.weight if self.affine else None
        b = self.bias if self.affine else None
        return _SyncBatchNormFunction.apply(input, w, b, mean, invstd, total, group)

    @classmethod
    def convert_sync_batchnorm(cls, module: torch.nn.Module, process_group: Any = None) -> torch.nn.Module:
        """Replace every ``BatchNorm*d`` in ``module`` (recursively) by this class, sharing parameters and buffers."""
        out = module
        if isinstance(module, torch.nn.modules.batchnorm._BatchNorm) and not isinstance(module, SyncBatchNorm):
            out = cls(module.num_features, module.eps, module.momentum, module.affine, module.track_running_stats,
                      process_group=process_group)
            if module.affine:
                out.weight, out.bias = module.weight, module.bias
            out.running_mean, out.running_var = module.running_mean, module.running_var
            out.num_batches_tracked = module.num_batches_tracked
            if hasattr(module, "qconfig"):
                out.qconfig = module.qconfig
        for name, child in module.named_children():
            out.add_module(name, cls.convert_sync_batchnorm(child, process_group))
        return out
