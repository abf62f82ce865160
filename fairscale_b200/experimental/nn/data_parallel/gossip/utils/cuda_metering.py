"""Named CUDA-event timers with a mean / std report (parity: .../gossip/utils/cuda_metering.py:27-115)."""

from __future__ import annotations

from abc import ABC, abstractmethod
from collections import defaultdict, deque
from functools import partial
import statistics
from typing import ClassVar, Deque, Dict, Optional

import torch

MAX_LEN_DEQUEUE = 10**4
deque_with_max_len_fixed = partial(deque, maxlen=MAX_LEN_DEQUEUE)


def create_and_record_event() -> torch.cuda.Event:
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    return ev


class EventRecorder(ABC):
    @abstractmethod
    def stop(self) -> None:
        ...


def create_event_recorder(event_name: str, dummy: bool = False) -> EventRecorder:
    return DummyCudaEventRecorder() if dummy or not torch.cuda.is_available() else CudaEventRecorder(event_name)


class CudaEventRecorder(EventRecorder):
    """Records a start event when created and an end event on ``stop()``; elapsed times are resolved lazily (no
    synchronisation in the training loop) when a report is requested."""

    event_recorders: ClassVar[Dict[str, Deque["CudaEventRecorder"]]] = defaultdict(deque_with_max_len_fixed)  # type: ignore[arg-type]
    all_event_recorders: ClassVar[Dict[str, Deque["CudaEventRecorder"]]] = defaultdict(deque_with_max_len_fixed)  # type: ignore[arg-type]

    def __init__(self, event_name: str) -> None:
        self.event_name = event_name
        self.start_event = create_and_record_event()
        self.end_event: Optional[torch.cuda.Event] = None
        CudaEventRecorder.event_recorders[event_name].append(self)
        CudaEventRecorder.all_event_recorders[event_name].append(self)

    def stop(self) -> None:
        self.end_event = create_and_record_event()

    def find_time_elapsed(self) -> float:
        if self.end_event is None:
            raise Exception(f"stopEvent was not called for event with name {self.event_name}")
        self.end_event.synchronize()
        return self.start_event.elapsed_time(self.end_event)

    @classmethod
    def reset(cls) -> None:
        cls.event_recorders = defaultdict(deque_with_max_len_fixed)  # type: ignore[arg-type]

    @classmethod
    def get_common_timings(cls, event_recorders: Dict[str, Deque["CudaEventRecorder"]], description: str) -> str:
        lines = [f"{description}:"]
        for name in sorted(event_recorders):
            times = [r.find_time_elapsed() for r in event_recorders[name]]
            std = statistics.pstdev(times) if len(times) > 1 else 0.0
            lines.append(f"{name} = {statistics.mean(times)} +/- {std}")
        return "\n".join(lines) + "\n"

    @classmethod
    def get_all_timings(cls) -> str:
        """Statistics of every timing recorded since the process started."""
        return cls.get_common_timings(cls.all_event_recorders, "All timings")

    @classmethod
    def get_timings(cls) -> str:
        """Report since the last ``reset()`` followed by the report over the whole run."""
        out = cls.get_common_timings(cls.event_recorders, "Timings since last reset")
        out += cls.get_common_timings(cls.all_event_recorders, "All timings")
        return out


class DummyCudaEventRecorder(EventRecorder):
    def stop(self) -> None:
        pass
