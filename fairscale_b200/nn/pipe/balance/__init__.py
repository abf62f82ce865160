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
    """Layers per partition when consecutive layers with these costs are cut into ``partitions`` blocks of similar cost."""
    return list(map(len, blockpartition.solve(cost, partitions)))


def _on(device: Device) -> torch.device:
    return device if isinstance(device, torch.device) else torch.device(device)


def balance_by_time(partitions: int, module: nn.Sequential, sample: TensorOrTensors, *, timeout: float = 1.0,
                    device: Device = torch.device("cuda")) -> List[int]:
    """Cut so that every partition takes about the same forward + backward time on ``sample`` (profiled for ``timeout`` s)."""
    return balance_cost(profile_times(module, sample, timeout, _on(device)), partitions)


def balance_by_size(partitions: int, module: nn.Sequential, input: TensorOrTensors, *, chunks: int = 1, param_scale: float = 2.0,
                    device: Device = torch.device("cuda")) -> List[int]:
    """Cut by memory: activations of one of ``chunks`` micro-batches plus ``param_scale`` x parameter bytes (2 for SGD: weight +
    gradient; 4 for Adam: two moments more)."""
    return balance_cost(profile_sizes(module, input, chunks, param_scale, _on(device)), partitions)
