"""Autograd-aware collectives between "replicated" and "tensor-parallel" regions.

Parity: fairscale/nn/model_parallel/mappings.py:30-156 (the Megatron f / g operators and the
scatter / gather pair).  Collectives go through :mod:`fairscale_b200.parallel.comm`, i.e. the NVLink
kernels when a symmetric workspace exists for the model-parallel group and NCCL / gloo otherwise.
The gather along the last dimension is :func:`fairscale_b200.parallel.comm.all_gather_last_dim`: over NVLink the pulling
kernel writes every rank's slice straight into its column window of the output; over NCCL / gloo it is one all-gather
along a leading axis plus one transposing copy (the reference uses ``all_gather`` into a list + ``torch.cat``).
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from ...parallel import comm
from .initialize import get_model_parallel_group
from .utils import split_tensor_along_last_dim


def _reduce(ctx: Any, input_: torch.Tensor) -> torch.Tensor:
    """In-place sum over the model-parallel group."""
    group = get_model_parallel_group()
    if ctx is not None:
        ctx.mark_dirty(input_)
    if dist.get_world_size(group=group) == 1:
        return input_
    comm.all_reduce(input_, group=group)
    return input_


def _split(input_: torch.Tensor) -> torch.Tensor:
    """Keep this rank's slice of the last dimension."""
    group = get_model_parallel_group()
    world = dist.get_world_size(group=group)
    if world == 1:
        return input_
    return split_tensor_along_last_dim(input_, world)[dist.get_rank(group=group)].contiguous()


def _gather(input_: torch.Tensor) -> torch.Tensor:
    """Concatenate every rank's tensor along the last dimension."""
    group = get_model_parallel_group()
    world = dist.get_world_size(group=group)
    if world == 1:
        return input_
    return comm.all_gather_last_dim(input_, group=group)


class _CopyToModelParallelRegion(torch.autograd.Function):
    """Identity forward, all-reduce backward (Megatron's ``f``)."""

    @staticmethod
    def forward(ctx, input_):  # type: ignore[override]
        return input_

    @staticmethod
    def backward(ctx, grad_output):  # type: ignore[override]
        return _reduce(None, grad_output)


class _ReduceFromModelParallelRegion(torch.autograd.Function):
    """All-reduce forward, identity backward (Megatron's ``g``)."""

    @staticmethod
    def forward(ctx, input_):  # type: ignore[override]
        return _reduce(ctx, input_)

    @staticmethod
    def backward(ctx, grad_output):  # type: ignore[override]
        return grad_output


class _ScatterToModelParallelRegion(torch.autograd.Function):
    """Slice forward, gather backward."""

    @staticmethod
    def forward(ctx, input_):  # type: ignore[override]
        return _split(input_)

    @staticmethod
    def backward(ctx, grad_output):  # type: ignore[override]
        return _gather(grad_output)


class _GatherFromModelParallelRegion(torch.autograd.Function):
    """Gather forward, slice backward."""

    @staticmethod
    def forward(ctx, input_):  # type: ignore[override]
        return _gather(input_)

    @staticmethod
    def backward(ctx, grad_output):  # type: ignore[override]
        return _split(grad_output)


def copy_to_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    return _CopyToModelParallelRegion.apply(input_)


def reduce_from_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    return _ReduceFromModelParallelRegion.apply(input_)


def scatter_to_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    return _ScatterToModelParallelRegion.apply(input_)


def gather_from_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    return _GatherFromModelParallelRegion.apply(input_)
