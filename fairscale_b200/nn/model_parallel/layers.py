"""Megatron-style tensor-parallel layers.

API parity with fairscale/nn/model_parallel/layers.py:44-387: ``VocabParallelEmbedding``,
``ParallelEmbedding``, ``ColumnParallelLinear``, ``RowParallelLinear`` with identical constructor
signatures, weight shapes (``[out/p, in]`` / ``[out, in/p]``), master-weight initialisation (the full
weight is drawn from the same RNG on every rank and sliced, so a tensor-parallel model starts equal to the
dense model under the same seed) and zero-initialised, unsharded-after-reduce bias handling.

On CUDA bf16 inputs the local products run on the tcgen05 GEMM; with ``sequence_parallel=True`` a
``ColumnParallelLinear`` consumes sequence-sharded input through the fused all-gather->GEMM kernel and a
``RowParallelLinear`` produces sequence-sharded output through the fused GEMM->reduce-scatter kernel
(:mod:`fairscale_b200.parallel.fused_tp`), replacing the two all-reduces per layer of the reference
(mappings.py:42) by NVLink traffic that overlaps the tiles' math.
"""

from __future__ import annotations

import os
from typing import Callable, Optional

import torch
import torch.nn.functional as F
import torch.nn.init as init
from torch.nn.parameter import Parameter

from ...ops import gemm as _gemm
from .initialize import get_model_parallel_group, get_model_parallel_rank, get_model_parallel_world_size
from .mappings import (
    copy_to_model_parallel_region,
    gather_from_model_parallel_region,
    reduce_from_model_parallel_region,
    scatter_to_model_parallel_region,
)
from .utils import VocabUtility, divide_and_check_no_remainder


__all__ = [
    "ColumnParallelLinear",
    "RowParallelLinear",
    "VocabParallelEmbedding",
    "ParallelEmbedding",
]


def _local_linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
        return _gemm.linear(x, w, b)
    return F.linear(x, w, b)


_GPU_DRAW_MIN_NUMEL = 1 << 24  # full weights of at least this many elements are drawn on the GPU


def _initialize_affine_weight(
    weight: torch.Tensor,
    out_features: int,
    in_features: int,
    per_partition_size: int,
    partition_dim: int,
    init_method: Callable[[torch.Tensor], torch.Tensor],
    stride: int = 1,
    return_master_weight: bool = False,
) -> Optional[torch.Tensor]:
    """Draw the full ``[out, in]`` weight with ``init_method`` on every rank and keep this rank's slices.

    With ``stride > 1`` the partitioned dimension is cut into ``stride * world`` pieces and rank ``r`` keeps
    pieces ``r, r + world, …`` (layout of fused QKV / gate-up projections).
    """
    world = get_model_parallel_world_size()
    if world == 1:
        init_method(weight)
        return weight if return_master_weight else None
    # The full weight is drawn where it is cheapest: large ones on this rank's GPU when there is one (a CPU draw of a
    # 7 B-parameter model takes minutes per rank), small ones on the CPU as in the reference (same values as a dense layer
    # initialised with the same seed).  Every rank uses the same device type and seed,
    # so the result is still independent of the model-parallel world size.
    big = out_features * in_features >= _GPU_DRAW_MIN_NUMEL
    draw_on = torch.device("cuda", torch.cuda.current_device()) if (big and torch.cuda.is_available()) else torch.device("cpu")
    master = torch.empty(out_features, in_features, dtype=weight.dtype, requires_grad=False, device=draw_on)
    init_method(master)
    if not return_master_weight and master.device != weight.device:
        piece = divide_and_check_no_remainder(per_partition_size, stride)
        mine = torch.split(master, piece, dim=partition_dim)[get_model_parallel_rank()::world]
        with torch.no_grad():
            weight.copy_(torch.cat(mine, dim=partition_dim))  # only this rank's slice crosses to the weight's device
        return None
    master = master.to(weight.device)
    piece = divide_and_check_no_remainder(per_partition_size, stride)
    pieces = torch.split(master, piece, dim=partition_dim)
    mine = pieces[get_model_parallel_rank()::world]
    with torch.no_grad():
        weight.copy_(torch.cat(mine, dim=partition_dim))
    return master if return_master_weight else None


class _ShardedEmbedding(torch.nn.Module):
    """What both sharded embeddings take over from ``torch.nn.Embedding``: its settings, and the library lookup that honours
    all of them."""

    weight: Parameter

    def _keep_settings(self, num_embeddings, embedding_dim, padding_idx, max_norm, norm_type, scale_grad_by_freq, sparse) -> None:
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx, self.max_norm, self.norm_type = padding_idx, max_norm, norm_type
        self.scale_grad_by_freq, self.sparse = scale_grad_by_freq, sparse
        self._weight = None

    def _is_plain_lookup(self) -> bool:
        """No setting asks for more than ``weight[ids]``."""
        return self.padding_idx is None and self.max_norm is None and not (self.scale_grad_by_freq or self.sparse)

    def _torch_lookup(self, ids: torch.Tensor, padding_idx: Optional[int]) -> torch.Tensor:
        return F.embedding(ids, self.weight, padding_idx, self.max_norm, self.norm_type, self.scale_grad_by_freq, self.sparse)


class VocabParallelEmbedding(_ShardedEmbedding):
    """Embedding whose vocabulary rows are split across the model-parallel group.

    Tokens outside the local range contribute zeros; the partial results are summed with an all-reduce.
    """

    def __init__(
        self,
        num_embeddings: int,
        embedding_dim: int,
        padding_idx: Optional[int] = None,
        max_norm: Optional[float] = None,
        norm_type: float = 2.0,
        scale_grad_by_freq: bool = False,
        sparse: bool = False,
        init_method: Callable[[torch.Tensor], torch.Tensor] = init.xavier_normal_,
    ) -> None:
        super().__init__()
        self._keep_settings(num_embeddings, embedding_dim, padding_idx, max_norm, norm_type, scale_grad_by_freq, sparse)
        self.vocab_start_index, self.vocab_end_index = VocabUtility.vocab_range_from_global_vocab_size(
            num_embeddings, get_model_parallel_rank(), get_model_parallel_world_size()
        )
        self.num_embeddings_per_partition = self.vocab_end_index - self.vocab_start_index
        self.weight = Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim))
        _initialize_affine_weight(self.weight, num_embeddings, embedding_dim, self.num_embeddings_per_partition, 0, init_method)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        if self._is_plain_lookup() and input_.is_cuda and self.weight.dtype == torch.bfloat16 and self.embedding_dim % 8 == 0:
            from ...ops.embedding import embedding

            # the kernel masks out-of-range ids itself (no index clone / masked writes)
            partial = embedding(input_, self.weight, None, 1.0, self.vocab_start_index)
        else:
            outside = (input_ < self.vocab_start_index) | (input_ >= self.vocab_end_index)
            local = input_.clone() - self.vocab_start_index
            local[outside] = 0
            # padding_idx names a row of the whole vocabulary: only the rank that holds the row passes it on, renumbered
            pad = self.padding_idx
            if pad is not None:
                pad = pad + self.num_embeddings if pad < 0 else pad
                pad = pad - self.vocab_start_index if self.vocab_start_index <= pad < self.vocab_end_index else None
            partial = self._torch_lookup(local, pad)
            partial[outside, :] = 0.0
        return reduce_from_model_parallel_region(partial)


class ParallelEmbedding(_ShardedEmbedding):
    """Embedding whose embedding dimension is split across the model-parallel group (outputs are gathered)."""

    def __init__(
        self,
        num_embeddings: int,
        embedding_dim: int,
        padding_idx: Optional[int] = None,
        max_norm: Optional[float] = None,
        norm_type: float = 2.0,
        scale_grad_by_freq: bool = False,
        sparse: bool = False,
        init_method: Callable[[torch.Tensor], torch.Tensor] = init.xavier_normal_,
        keep_master_weight_for_test: bool = False,
    ) -> None:
        super().__init__()
        self._keep_settings(num_embeddings, embedding_dim, padding_idx, max_norm, norm_type, scale_grad_by_freq, sparse)
        world = get_model_parallel_world_size()
        self.embedding_dim_per_partition = divide_and_check_no_remainder(embedding_dim, world)
        self.weight = Parameter(torch.empty(num_embeddings, self.embedding_dim_per_partition))
        _initialize_affine_weight(self.weight, num_embeddings, embedding_dim, self.embedding_dim_per_partition, 1,
                                  init_method, stride=1, return_master_weight=False)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        input_parallel = copy_to_model_parallel_region(input_)
        if self._is_plain_lookup() and input_.is_cuda and self.weight.dtype == torch.bfloat16 and self.embedding_dim_per_partition % 8 == 0:
            from ...ops.embedding import embedding

            local = embedding(input_parallel, self.weight)  # native gather kernel; its backward scatters into the slice
        else:
            local = self._torch_lookup(input_parallel, self.padding_idx)
        return gather_from_model_parallel_region(local)


class ColumnParallelLinear(torch.nn.Module):
    """``Y = X A^T + b`` with the output features of ``A`` split across ranks: rank i computes ``Y_i = X A_i^T``.

    ``gather_output=True`` all-gathers the ``Y_i`` so every rank holds ``Y``.  ``sequence_parallel=True``
    (extension) expects ``X`` sharded along the token dimension and gathers it inside the GEMM kernel.
    """

    def __init__(
        self,
        in_features: int,
        out_features: int,
        bias: bool = True,
        gather_output: bool = True,
        init_method: Callable[[torch.Tensor], torch.Tensor] = init.xavier_normal_,
        stride: int = 1,
        keep_master_weight_for_test: bool = False,
        sequence_parallel: bool = False,
    ) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.gather_output = gather_output
        self.sequence_parallel = sequence_parallel
        world = get_model_parallel_world_size()
        self.output_size_per_partition = divide_and_check_no_remainder(out_features, world)
        self.weight = Parameter(torch.empty(self.output_size_per_partition, in_features))
        if bias:
            self.bias = Parameter(torch.zeros(self.output_size_per_partition))
        else:
            self.register_parameter("bias", None)
        self.master_weight = _initialize_affine_weight(
            self.weight, out_features, in_features, self.output_size_per_partition, 0, init_method, stride=stride,
            return_master_weight=keep_master_weight_for_test,
        )

    def get_master_weight(self) -> torch.Tensor:
        return gather_from_model_parallel_region(self.weight.data.transpose(0, 1)).transpose_(0, 1)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        if self.sequence_parallel:
            from ...parallel.fused_tp import all_gather_linear

            out = all_gather_linear(input_, self.weight, self.bias, get_model_parallel_group())
        else:
            out = _local_linear(copy_to_model_parallel_region(input_), self.weight, self.bias)
        return gather_from_model_parallel_region(out) if self.gather_output else out


class RowParallelLinear(torch.nn.Module):
    """``Y = X A^T + b`` with the input features split: rank i holds ``A_i`` and ``X_i``; ``Y = sum_i X_i A_i^T``.

    The bias is not sharded and is added once, after the reduction.  ``sequence_parallel=True`` (extension)
    returns ``Y`` sharded along the token dimension through the fused GEMM->reduce-scatter kernel.
    """

    def __init__(
        self,
        in_features: int,
        out_features: int,
        bias: bool = True,
        input_is_parallel: bool = False,
        init_method: Callable[[torch.Tensor], torch.Tensor] = init.xavier_normal_,
        stride: int = 1,
        keep_master_weight_for_test: bool = False,
        sequence_parallel: bool = False,
    ):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.input_is_parallel = input_is_parallel
        self.sequence_parallel = sequence_parallel
        world = get_model_parallel_world_size()
        self.input_size_per_partition = divide_and_check_no_remainder(in_features, world)
        self.weight = Parameter(torch.empty(out_features, self.input_size_per_partition))
        if bias:
            self.bias = Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)
        self.master_weight = _initialize_affine_weight(
            self.weight, out_features, in_features, self.input_size_per_partition, 1, init_method, stride=stride,
            return_master_weight=keep_master_weight_for_test,
        )

    def get_master_weight(self) -> torch.Tensor:
        return gather_from_model_parallel_region(self.weight.data)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        x = input_ if self.input_is_parallel else scatter_to_model_parallel_region(input_)
        if self.sequence_parallel:
            from ...parallel.fused_tp import linear_reduce_scatter

            return linear_reduce_scatter(x, self.weight, self.bias, get_model_parallel_group())
        if os.environ.get("FSB200_FUSED_ROW_ALLREDUCE", "0") == "1":
            # opt-in: fused GEMM -> reduce-scatter + all-gather of the reduced rows instead of GEMM + all-reduce
            from ...parallel.fused_tp import linear_all_reduce

            return linear_all_reduce(x, self.weight, self.bias, get_model_parallel_group())
        partial = _local_linear(x, self.weight, None)
        out = reduce_from_model_parallel_region(partial)
        return out if self.bias is None else out + self.bias
