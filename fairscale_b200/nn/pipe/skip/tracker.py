"""Where skippable modules put and find their skip tensors while a model runs.

Outside a pipeline the tracker is a dictionary.  Inside one, every micro-batch has a :class:`StageSkipTracker`: skip
tensors that stay within the running partition still go through the dictionary, while routed ones (see
``skip/layout.py``) are taken from the stage's *inbox* (filled by the pipeline from the stage's extra inputs) and put into
its *outbox* (returned by the pipeline as the stage's extra outputs).  Between stages the pipeline keeps a routed
tensor in ``in_transit`` on the device that produced it.  Interface of fairscale/nn/pipe/skip/tracker.py:38-211.
"""

from __future__ import annotations

import threading
from contextlib import contextmanager
from typing import Dict, Generator, List, Optional, Tuple

from torch import Tensor

from ..copy import Copy, Wait
from ..microbatch import Batch
from ..stream import AbstractStream
from .layout import SkipKey, SkipLayout
from .namespace import Namespace

__all__: List[str] = []


class SkipTracker:
    """Dictionary tracker: what a skippable module sees when no pipeline is driving it."""

    def __init__(self) -> None:
        self.tensors: Dict[SkipKey, Optional[Tensor]] = {}

    @property
    def index(self) -> int:
        return 0

    def save(self, batch: Batch, ns: Optional[Namespace], name: str, tensor: Optional[Tensor]) -> None:
        self.tensors[(ns, name)] = tensor

    def load(self, batch: Batch, ns: Optional[Namespace], name: str) -> Optional[Tensor]:
        return self.tensors.pop((ns, name))  # KeyError: popped before stashed

    def copy(self, batch: Batch, prev_stream: AbstractStream, next_stream: AbstractStream, ns: Optional[Namespace], name: str) -> None:
        raise TypeError("copy is not supported for non-portal skip tensors")


class StageSkipTracker(SkipTracker):
    """Tracker of one micro-batch inside a pipeline."""

    def __init__(self, skip_layout: SkipLayout, index: int = 0) -> None:
        super().__init__()
        self.skip_layout = skip_layout
        self._index = index
        self.inbox: Dict[SkipKey, Optional[Tensor]] = {}       # routed tensors delivered to the running stage
        self.outbox: Dict[SkipKey, Optional[Tensor]] = {}      # routed tensors stashed by the running stage
        self.in_transit: Dict[SkipKey, Optional[Tensor]] = {}  # routed tensors between their two stages

    @property
    def index(self) -> int:
        return self._index

    def save(self, batch: Batch, ns: Optional[Namespace], name: str, tensor: Optional[Tensor]) -> None:
        if self.skip_layout.requires_copy(ns, name):
            self.outbox[(ns, name)] = tensor
        else:
            super().save(batch, ns, name, tensor)

    def load(self, batch: Batch, ns: Optional[Namespace], name: str) -> Optional[Tensor]:
        if self.skip_layout.requires_copy(ns, name):
            return self.inbox.pop((ns, name))
        return super().load(batch, ns, name)

    def copy(self, batch: Batch, prev_stream: AbstractStream, next_stream: AbstractStream, ns: Optional[Namespace], name: str) -> None:
        """Bring the routed tensor ``(ns, name)`` from the device of ``prev_stream`` to the device of ``next_stream``
        (asynchronously, on those copy streams); it stays in ``in_transit`` until its stage starts."""
        key = (ns, name)
        tensor = self.in_transit.get(key)
        if tensor is None:
            return  # stashed as None: nothing to move
        (moved,) = Copy.apply(prev_stream, next_stream, tensor)
        self.in_transit[key] = moved if moved.is_floating_point() else moved.detach()

    def deliver(self, keys: List[SkipKey], copy_stream: AbstractStream, compute_stream: AbstractStream) -> Tuple[List[SkipKey], List[Tensor]]:
        """Take the tensors for input ports ``keys`` out of ``in_transit`` after making ``compute_stream`` wait for
        their copies on ``copy_stream``.  Returns the keys that carry a tensor and those tensors; a key whose value was
        stashed as ``None`` goes to the inbox directly and needs no port."""
        carried: List[SkipKey] = []
        for key in keys:
            if self.in_transit.get(key) is None:
                self.in_transit.pop(key, None)
                self.inbox[key] = None
            else:
                carried.append(key)
        if not carried:
            return [], []
        waited = Wait.apply(copy_stream, compute_stream, *[self.in_transit.pop(k) for k in carried])
        return carried, [t if t.is_floating_point() else t.detach() for t in waited]


# the reference's (misspelt) name for the pipeline tracker
SkipTrackerThroughPotals = StageSkipTracker


class _Current(threading.local):
    tracker: Optional[SkipTracker] = None


_current = _Current()


@contextmanager
def use_skip_tracker(skip_tracker: SkipTracker) -> Generator[None, None, None]:
    """Make ``skip_tracker`` the one skippable modules of this thread talk to."""
    saved, _current.tracker = _current.tracker, skip_tracker
    try:
        yield
    finally:
        _current.tracker = saved


def current_skip_tracker() -> SkipTracker:
    if _current.tracker is None:
        _current.tracker = SkipTracker()
    return _current.tracker
