"""Named CUDA-event timers with a mean / std report (interface of .../gossip/utils/cuda_metering.py:27-115).

A recorder stamps a start event when it is created and an end event on ``stop()``.  Nothing synchronises in the training
loop: elapsed times are resolved only when a report is asked for.  Recorders are kept in two registries of bounded
length per name - one that ``reset()`` empties (``event_recorders``) and one that covers the whole run
(``all_event_recorders``).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from collections import defaultdict, deque
import statistics
from typing import ClassVar, Deque, Dict, Optional

import torch

MAX_LEN_DEQUEUE = 10**4


def deque_with_max_len_fixed() -> "Deque[CudaEventRecorder]":
    return deque(maxlen=MAX_LEN_DEQUEUE)


def _registry() -> "Dict[str, Deque[CudaEventRecorder]]":
    return defaultdict(deque_with_max_len_fixed)


def create_and_record_event() -> torch.cuda.Event:
    """A timing event stamped on the current stream."""
    stamp = torch.cuda.Event(enable_timing=True)
    stamp.record()
    return stamp


class EventRecorder(ABC):
    @abstractmethod
    def stop(self) -> None:
        ...


class DummyCudaEventRecorder(EventRecorder):
    """Stands in where timing is off or there is no GPU."""

    def stop(self) -> None:
        return None


class CudaEventRecorder(EventRecorder):
    event_recorders: ClassVar[Dict[str, Deque["CudaEventRecorder"]]] = _registry()
    all_event_recorders: ClassVar[Dict[str, Deque["CudaEventRecorder"]]] = _registry()

    def __init__(self, event_name: str) -> None:
        self.event_name = event_name
        self.start_event = create_and_record_event()
        self.end_event: Optional[torch.cuda.Event] = None
        for registry in (CudaEventRecorder.event_recorders, CudaEventRecorder.all_event_recorders):
            registry[event_name].append(self)

    def stop(self) -> None:
        self.end_event = create_and_record_event()

    def find_time_elapsed(self) -> float:
        """Milliseconds between creation and ``stop()``; waits for the end event."""
        if self.end_event is None:
            raise Exception(f"stopEvent was not called for event with name {self.event_name}")
        self.end_event.synchronize()
        return self.start_event.elapsed_time(self.end_event)

    @classmethod
    def reset(cls) -> None:
        cls.event_recorders = _registry()

    @staticmethod
    def _line(name: str, recorders: "Deque[CudaEventRecorder]") -> str:
        ms = [r.find_time_elapsed() for r in recorders]
        spread = statistics.pstdev(ms) if len(ms) > 1 else 0.0
        return f"{name} = {statistics.mean(ms)} +/- {spread}"

    @classmethod
    def get_common_timings(cls, event_recorders: Dict[str, Deque["CudaEventRecorder"]], description: str) -> str:
        body = [cls._line(name, event_recorders[name]) for name in sorted(event_recorders)]
        return "\n".join([f"{description}:"] + body) + "\n"

    @classmethod
    def get_all_timings(cls) -> str:
        """Statistics of every timing recorded since the process started."""
        return cls.get_common_timings(cls.all_event_recorders, "All timings")

    @classmethod
    def get_timings(cls) -> str:
        """Report since the last ``reset()`` followed by the report over the whole run."""
        return cls.get_common_timings(cls.event_recorders, "Timings since last reset") + cls.get_all_timings()


def create_event_recorder(event_name: str, dummy: bool = False) -> EventRecorder:
    if dummy or not torch.cuda.is_available():
        return DummyCudaEventRecorder()
    return CudaEventRecorder(event_name)
