"""Helpers for tensor parallel layers (names of fairscale/nn/model_parallel/utils.py:27-78)."""

from __future__ import annotations

from typing import Tuple

import torch


def divide_and_check_no_remainder(numerator: int, denominator: int) -> int:
    """``numerator / denominator`` when that is a whole number, an assertion error otherwise."""
    quotient, remainder = divmod(numerator, denominator)
    assert remainder == 0, f"{numerator} is not divisible by {denominator}"
    return quotient


def ensure_divisibility(numerator: int, denominator: int) -> None:
    divide_and_check_no_remainder(numerator, denominator)


def split_tensor_along_last_dim(
    tensor: torch.Tensor, num_partitions: int, contiguous_split_chunks: bool = False
) -> Tuple[torch.Tensor, ...]:
    """``num_partitions`` equal pieces of the last dimension: views, or copies with ``contiguous_split_chunks``."""
    width = divide_and_check_no_remainder(tensor.size(-1), num_partitions)
    pieces = tensor.split(width, dim=-1)
    return tuple(p.contiguous() for p in pieces) if contiguous_split_chunks else pieces


class VocabUtility:
    """Which ``[first, last)`` slice of the vocabulary a rank owns when it is dealt out in equal consecutive blocks."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition_vocab_size: int, rank: int, world_size: int) -> Tuple[int, int]:
        return rank * per_partition_vocab_size, (rank + 1) * per_partition_vocab_size

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab_size: int, rank: int, world_size: int) -> Tuple[int, int]:
        block = divide_and_check_no_remainder(global_vocab_size, world_size)
        return VocabUtility.vocab_range_from_per_partition_vocab_size(block, rank, world_size)
