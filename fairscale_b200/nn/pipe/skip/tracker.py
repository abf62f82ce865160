"""Per-micro-batch registry of live skip tensors (parity: fairscale/nn/pipe/skip/tracker.py:38-211)."""

from __future__ import annotations

import threading
from contextlib import contextmanager
from typing import Dict, Generator, List, Optional, Tuple

from torch import Tensor

from ..checkpoint import is_checkpointing
from ..dependency import fork, join
from ..microbatch import Batch
from ..stream import AbstractStream
from .layout import SkipLayout
from .namespace import Namespace
from .portal import Portal

__all__: List[str] = []


class SkipTracker:
    """Plain dictionary tracker used outside ``Pipe`` (skippable modules then behave like ordinary modules)."""

    def __init__(self) -> None:
        self.tensors: Dict[Tuple[Namespace, str], Optional[Tensor]] = {}

    def save(self, batch: Batch, ns: Namespace, name: str, tensor: Optional[Tensor]) -> None:
        self.tensors[(ns, name)] = tensor

    def load(self, batch: Batch, ns: Namespace, name: str) -> Optional[Tensor]:
        return self.tensors.pop((ns, name))

    def copy(self, batch: Batch, prev_stream: AbstractStream, next_stream: AbstractStream, ns: Namespace, name: str) -> None:
        raise TypeError("copy is not supported for non-portal skip tensors")

    @property
    def index(self) -> int:
        return 0


class SkipTrackerThroughPotals(SkipTracker):
    """Tracker used by ``Pipe``: tensors that cross partitions travel through :class:`Portal` objects."""

    def __init__(self, skip_layout: SkipLayout, index: int = 0) -> None:
        super().__init__()
        self.skip_layout = skip_layout
        self.portals: Dict[Tuple[Namespace, str], Portal] = {}
        self.__index = index

    @property
    def index(self) -> int:
        return self.__index

    def save(self, batch: Batch, ns: Namespace, name: str, tensor: Optional[Tensor]) -> None:
        if not self.skip_layout.requires_copy(ns, name):
            super().save(batch, ns, name, tensor)
            return
        if (ns, name) not in self.portals:
            # requested once by the copy + once by the pop, plus once more by the recomputed pop when checkpointing
            life = 3 if is_checkpointing() else 2
            portal = Portal(tensor, life, batch.index)
            portal.ns_name = (ns, name)
            self.portals[(ns, name)] = portal
        else:
            # the stash re-executes during recomputation: only blue() below will take the tensor
            portal = self.portals[(ns, name)]
            portal.put_tensor(tensor, 1)
        phony = portal.blue()
        batch[0] = join(batch[0], phony)

    def load(self, batch: Batch, ns: Namespace, name: str) -> Optional[Tensor]:
        if not self.skip_layout.requires_copy(ns, name):
            return super().load(batch, ns, name)
        portal = self.portals[(ns, name)]
        batch[0], phony = fork(batch[0])
        return portal.orange(phony)

    def copy(self, batch: Batch, prev_stream: AbstractStream, next_stream: AbstractStream, ns: Namespace, name: str) -> None:
        assert self.skip_layout.requires_copy(ns, name)
        batch[0], phony = fork(batch[0])
        portal = self.portals[(ns, name)]
        phony = portal.copy(prev_stream, next_stream, phony)
        batch[0] = join(batch[0], phony)


class _Local(threading.local):
    def __init__(self) -> None:
        self.skip_tracker: Optional[SkipTracker] = None


thread_local = _Local()


@contextmanager
def use_skip_tracker(skip_tracker: SkipTracker) -> Generator[None, None, None]:
    prev = thread_local.skip_tracker
    thread_local.skip_tracker = skip_tracker
    try:
        yield
    finally:
        thread_local.skip_tracker = prev


def current_skip_tracker() -> SkipTracker:
    if thread_local.skip_tracker is None:
        thread_local.skip_tracker = SkipTracker()
    return thread_local.skip_tracker
