"""Autograd-aware collectives between "replicated" and "tensor-parallel" regions.

Behaviour of fairscale/nn/model_parallel/mappings.py:30-156 (the Megatron f / g operators and the scatter / gather
pair), built from one table: each region operator is a (forward primitive, backward primitive) pair out of the three
primitives ``identity``, ``sum over the group``, ``slice / concatenate the last dimension``, and one generic autograd
function applies a pair.  Collectives go through :mod:`fairscale_b200.parallel.comm`, i.e. the NVLink kernels when a
symmetric workspace exists for the model-parallel group and NCCL / gloo otherwise.  The gather along the last dimension
is :func:`fairscale_b200.parallel.comm.all_gather_last_dim`: over NVLink the pulling kernel writes every rank's slice
straight into its column window of the output; over NCCL / gloo it is one all-gather along a leading axis plus one
transposing copy (the reference uses ``all_gather`` into a list + ``torch.cat``).
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Tuple

import torch
import torch.distributed as dist

from ...parallel import comm
from .initialize import get_model_parallel_group
from .utils import split_tensor_along_last_dim

__all__ = [
    "copy_to_model_parallel_region",
    "reduce_from_model_parallel_region",
    "scatter_to_model_parallel_region",
    "gather_from_model_parallel_region",
]


Primitive = Callable[[torch.Tensor], torch.Tensor]


def _group_and_size() -> Tuple[Any, int]:
    group = get_model_parallel_group()
    return group, dist.get_world_size(group=group)


# ---------------------------------------------------------------------------------------------------------- primitives
def _identity(t: torch.Tensor) -> torch.Tensor:
    return t


def _sum_over_group(t: torch.Tensor) -> torch.Tensor:
    """In place: every rank ends up with the sum."""
    group, world = _group_and_size()
    if world > 1:
        comm.all_reduce(t, group=group)
    return t


def _own_slice(t: torch.Tensor) -> torch.Tensor:
    """This rank's slice of the last dimension."""
    group, world = _group_and_size()
    if world == 1:
        return t
    return split_tensor_along_last_dim(t, world)[dist.get_rank(group=group)].contiguous()


def _concat_slices(t: torch.Tensor) -> torch.Tensor:
    """Every rank's tensor side by side along the last dimension."""
    group, world = _group_and_size()
    if world == 1:
        return t
    return comm.all_gather_last_dim(t, group=group)


# the names the reference's helpers go by
_reduce = lambda ctx, t: _sum_over_group(t)  # noqa: E731
_split = _own_slice
_gather = _concat_slices

# operator -> (forward, backward, forward works in place)
_REGION_OPS: Dict[str, Tuple[Primitive, Primitive, bool]] = {
    "copy": (_identity, _sum_over_group, False),      # f: replicated activations enter a parallel region
    "reduce": (_sum_over_group, _identity, True),     # g: partial results leave it
    "scatter": (_own_slice, _concat_slices, False),
    "gather": (_concat_slices, _own_slice, False),
}


class _RegionOp(torch.autograd.Function):
    """Applies the forward primitive of ``kind``; its backward applies the paired primitive to the gradient."""

    @staticmethod
    def forward(ctx: Any, kind: str, t: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        fwd, _, in_place = _REGION_OPS[kind]
        ctx.kind = kind
        if in_place:
            if t.is_leaf and t.requires_grad:
                t = t.detach().clone()  # autograd refuses to overwrite a leaf that wants a gradient: reduce a copy
            else:
                ctx.mark_dirty(t)
        return fwd(t)

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor) -> Tuple[None, torch.Tensor]:  # type: ignore[override]
        return None, _REGION_OPS[ctx.kind][1](grad)


def copy_to_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    """Identity forward, all-reduce backward (Megatron's ``f``)."""
    return _RegionOp.apply("copy", input_)


def reduce_from_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    """All-reduce forward (in place), identity backward (Megatron's ``g``)."""
    return _RegionOp.apply("reduce", input_)


def scatter_to_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    """Slice of the last dimension forward, gather backward."""
    return _RegionOp.apply("scatter", input_)


def gather_from_model_parallel_region(input_: torch.Tensor) -> torch.Tensor:
    """Gather along the last dimension forward, slice backward."""
    return _RegionOp.apply("gather", input_)
