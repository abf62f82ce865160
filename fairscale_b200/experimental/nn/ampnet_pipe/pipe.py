"""AMPnetPipe: ``AsyncPipe`` driven by the asynchronous (stale-weight) event loop.

Parity: fairscale/experimental/nn/ampnet_pipe/pipe.py:20-73.
"""

from __future__ import annotations

from typing import Any

from torch import nn
from torch.optim.optimizer import Optimizer
from torch.utils.data import DataLoader

from ....nn.pipe import AsyncPipe
from .ampnet import AsyncAMPnetEventLoop

__all__ = ["AMPnetPipe"]


class AMPnetPipe(AsyncPipe):
    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)

    def interleave(self, lm_dataloader: DataLoader, criterion: nn.Module, optimizer: Optimizer, transform_logger_object: Any,
                   min_update_interval: int = 1, weight_prediction: bool = False) -> None:
        """Train one epoch.  Every stage iterates ``lm_dataloader`` (the head for inputs, the tail for targets, the
        others only to count batches)."""
        if self.partition is None:
            return
        n = len(self.balance)
        stop = {"always": 1 << 62, "except_last": 1 << 62, "never": 0}[self.checkpoint] if self.training else 0
        loop = AsyncAMPnetEventLoop(self.partition, self.rank, n, self.transport, min_update_interval, weight_prediction,
                                    stop, self.input_device, self.chunks)
        loop.run(lm_dataloader, criterion, optimizer, transform_logger_object)
