"""Per-rank driver of the event-loop schedule (parity: fairscale/nn/pipe/async_pipeline.py:26-88)."""

from __future__ import annotations

from typing import Any, List, Optional

from torch import Tensor

from .async_schedule import AsyncEventLoop, ModuleWrapper
from .messages import SendRecvTransport


class AsyncPipeline:
    """Owns this rank's layers and runs one mini-batch through :class:`AsyncEventLoop`.

    ``checkpoint_stop``: micro-batches below this index recompute their activations in backward.
    """

    def __init__(self, partitions: List[ModuleWrapper], group: Any, rank: int, transport: SendRecvTransport,
                 checkpoint_stop: int = 0) -> None:
        self.partitions = partitions
        self.group = group
        self.rank = rank
        self.transport = transport
        self.checkpoint_stop = checkpoint_stop
        self._loop: Optional[AsyncEventLoop] = None

    def run(self, training: bool, batches: Optional[List[Tensor]], chunks: int) -> Optional[List[Tensor]]:
        """Forward of ``chunks`` micro-batches; the tail rank gets the list of outputs back."""
        stop = self.checkpoint_stop if training else 0
        self._loop = AsyncEventLoop(self.partitions, self.rank, self.transport, stop)
        if not self.partitions:
            return None
        if self._loop.is_head:
            return self._loop.event_loop_head(batches or [], chunks)
        if self._loop.is_tail:
            return self._loop.event_loop_tail(chunks)
        self._loop.event_loop(chunks)
        return None

    def back(self) -> None:
        """This rank's share of backward (after ``loss.backward()`` on the tail)."""
        if self._loop is not None:
            self._loop.run_backward()

    def back_helper(self, output: Optional[List[Tensor]] = None) -> None:
        """Name used by the reference for the same step; ``output`` is not needed (the loop kept what it sent)."""
        self.back()
