"""Helpers for tensor parallel layers (parity: fairscale/nn/model_parallel/utils.py:27-78)."""

from __future__ import annotations

from typing import Tuple

import torch


def ensure_divisibility(numerator: int, denominator: int) -> None:
    assert numerator % denominator == 0, f"{numerator} is not divisible by {denominator}"


def divide_and_check_no_remainder(numerator: int, denominator: int) -> int:
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


def split_tensor_along_last_dim(
    tensor: torch.Tensor, num_partitions: int, contiguous_split_chunks: bool = False
) -> Tuple[torch.Tensor, ...]:
    """Equal split of the last dimension (views unless ``contiguous_split_chunks``)."""
    size = divide_and_check_no_remainder(tensor.size(-1), num_partitions)
    pieces = torch.split(tensor, size, dim=tensor.dim() - 1)
    if contiguous_split_chunks:
        return tuple(p.contiguous() for p in pieces)
    return pieces


class VocabUtility:
    """``[first, last)`` vocabulary range owned by a rank when the vocabulary is split evenly."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition_vocab_size: int, rank: int, world_size: int) -> Tuple[int, int]:
        first = rank * per_partition_vocab_size
        return first, first + per_partition_vocab_size

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab_size: int, rank: int, world_size: int) -> Tuple[int, int]:
        per = divide_and_check_no_remainder(global_vocab_size, world_size)
        return VocabUtility.vocab_range_from_per_partition_vocab_size(per, rank, world_size)
