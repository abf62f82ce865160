"""Automatic balancing of pipeline partitions (parity: fairscale/nn/pipe/balance/__init__.py:40-184)."""

from __future__ import annotations

from typing import Any, List, Tuple, Union

import torch
from torch import Tensor, nn

from . import blockpartition
from .profile import profile_sizes, profile_times

__all__ = ["balance_by_time", "balance_by_size"]

Device = Union[torch.device, int, str]
Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]


def balance_cost(cost: List[int], partitions: int) -> List[int]:
    return [len(block) for block in blockpartition.solve(cost, partitions)]


def balance_by_time(partitions: int, module: nn.Sequential, sample: TensorOrTensors, *, timeout: float = 1.0,
                    device: Device = torch.device("cuda")) -> List[int]:
    """Balance so that every partition takes about the same forward+backward time on ``sample``."""
    times = profile_times(module, sample, timeout, torch.device(device))
    return balance_cost(times, partitions)


def balance_by_size(partitions: int, module: nn.Sequential, input: TensorOrTensors, *, chunks: int = 1, param_scale: float = 2.0,
                    device: Device = torch.device("cuda")) -> List[int]:
    """Balance by memory: activations of one micro-batch plus ``param_scale`` x parameters (2 for SGD, 4 for Adam...)."""
    sizes = profile_sizes(module, input, chunks, param_scale, torch.device(device))
    return balance_cost(sizes, partitions)
