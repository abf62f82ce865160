"""One worker thread per pipeline device (parity: fairscale/nn/pipe/worker.py:48-176).

Kernel launches for different stages are issued from different host threads so that a slow Python section of
one stage does not delay the launches of the others.  Exceptions travel back to the caller as ``exc_info``.
"""

from __future__ import annotations

import sys
from contextlib import contextmanager
from queue import Empty, Queue
from threading import Thread
from types import TracebackType
from typing import TYPE_CHECKING, Callable, Dict, Generator, List, Optional, Tuple, Type, Union, cast

import torch

from .microbatch import Batch
from .stream import AbstractStream, use_device, use_stream

__all__: List[str] = []

ExcInfo = Tuple[Type[BaseException], BaseException, TracebackType]

if TYPE_CHECKING:
    InQueue = Queue[Optional["Task"]]
    OutQueue = Queue[Tuple[bool, Union[Tuple["Task", Batch], ExcInfo, None]]]
else:
    InQueue = Queue
    OutQueue = Queue


class Task:
    """A unit of stage work: ``compute`` runs in the worker thread on ``stream``; ``finalize`` (optional) runs
    in the main thread afterwards and is where early recomputation is wired into the graph."""

    def __init__(self, stream: AbstractStream, *, compute: Callable[[], Batch], finalize: Optional[Callable[[Batch], None]]) -> None:
        self.stream = stream
        self._compute = compute
        self._finalize = finalize
        self._grad_enabled = torch.is_grad_enabled()

    def compute(self) -> Batch:
        with use_stream(self.stream), torch.set_grad_enabled(self._grad_enabled):
            return self._compute()

    def finalize(self, batch: Batch) -> None:
        if self._finalize is None:
            return
        with use_stream(self.stream), torch.set_grad_enabled(self._grad_enabled):
            self._finalize(batch)


def worker(in_queue: InQueue, out_queue: OutQueue, device: torch.device) -> None:
    with use_device(device):
        while True:
            task = in_queue.get()
            if task is None:
                break
            try:
                batch = task.compute()
            except Exception:
                out_queue.put((False, cast(ExcInfo, sys.exc_info())))
                continue
            out_queue.put((True, (task, batch)))
    out_queue.put((False, None))


def create_workers(devices: List[torch.device]) -> Tuple[List[InQueue], List[OutQueue]]:
    """Start one daemon thread per distinct device; stages on the same device share a thread."""
    in_queues: List[InQueue] = []
    out_queues: List[OutQueue] = []
    by_device: Dict[torch.device, Tuple[InQueue, OutQueue]] = {}

    def normalize(device: torch.device) -> torch.device:
        if device.type == "cuda" and device.index is None:
            return torch.device("cuda", index=torch.cuda.current_device())
        if device.type == "cpu" and device.index is not None:
            return torch.device("cpu")
        return device

    for device in devices:
        device = normalize(device)
        if device not in by_device:
            in_q: InQueue = Queue()
            out_q: OutQueue = Queue()
            by_device[device] = (in_q, out_q)
            Thread(target=worker, args=(in_q, out_q, device), daemon=True).start()
        in_q, out_q = by_device[device]
        in_queues.append(in_q)
        out_queues.append(out_q)
    return in_queues, out_queues


def join_workers(in_queues: List[InQueue], out_queues: List[OutQueue]) -> None:
    """Ask every worker thread to stop and wait for its termination marker."""
    if sys.is_finalizing():
        return  # daemon threads are already gone at interpreter shutdown
    for q in set(in_queues):
        q.put(None)
    for q in set(out_queues):
        while True:
            try:
                ok, payload = q.get(timeout=2.0)
            except Empty:
                break  # the thread died with the interpreter or never started
            if not ok and payload is None:
                break  # termination marker; anything else is a stale result or exception record


@contextmanager
def spawn_workers(devices: List[torch.device]) -> Generator[Tuple[List[InQueue], List[OutQueue]], None, None]:
    try:
        in_queues, out_queues = create_workers(devices)
        yield in_queues, out_queues
    finally:
        join_workers(in_queues, out_queues)
