"""Optional helper threads for the single-process pipeline: one per device, fed through queues.

The pipeline issues all stages from one thread by default (kernel launches are asynchronous, so a second Python thread
adds nothing under the GIL unless a stage spends its time in host code that releases it).  With ``Pipeline(...,
threads=True)`` every stage's ``Task`` is handed to the thread of its device instead and the results come back in
order; exceptions travel back as ``sys.exc_info()`` triples.  Names and queue protocol as in
fairscale/nn/pipe/worker.py:48-176: an in-queue takes ``Task`` objects (``None`` stops the thread), the out-queue
yields ``(True, (task, batch))``, ``(False, exc_info)`` or, once after ``None``, ``(False, None)``.
"""

from __future__ import annotations

import sys
import threading
from contextlib import contextmanager
from queue import Empty, Queue
from types import TracebackType
from typing import Callable, Dict, Generator, Hashable, List, Optional, Tuple, Type

import torch

from .microbatch import Batch
from .stream import AbstractStream, use_device, use_stream

__all__: List[str] = []

ExcInfo = Tuple[Type[BaseException], BaseException, TracebackType]
InQueue = Queue
OutQueue = Queue


class Task:
    """Work of one stage on one micro-batch.  ``compute`` produces the stage's output on ``stream`` (possibly in a
    helper thread); ``finalize`` runs afterwards in the dispatching thread, on the same stream, and is where an early
    recomputation gets attached.  Both run under the autograd mode that was active when the task was made."""

    def __init__(self, stream: AbstractStream, *, compute: Callable[[], Batch], finalize: Optional[Callable[[Batch], None]]) -> None:
        self.stream = stream
        self._body = compute
        self._epilogue = finalize
        self._grad_mode = torch.is_grad_enabled()

    @contextmanager
    def _scope(self) -> Generator[None, None, None]:
        with use_stream(self.stream), torch.set_grad_enabled(self._grad_mode):
            yield

    def compute(self) -> Batch:
        with self._scope():
            return self._body()

    def finalize(self, batch: Batch) -> None:
        if self._epilogue is not None:
            with self._scope():
                self._epilogue(batch)


def worker(in_queue: InQueue, out_queue: OutQueue, device: torch.device) -> None:
    """Thread body: run tasks until ``None`` arrives, then post the termination marker."""
    with use_device(device):
        for task in iter(in_queue.get, None):
            try:
                out_queue.put((True, (task, task.compute())))
            except Exception:
                out_queue.put((False, sys.exc_info()))
    out_queue.put((False, None))


def _device_key(device: torch.device) -> Hashable:
    device = torch.device(device)
    if device.type == "cuda":
        return ("cuda", torch.cuda.current_device() if device.index is None else device.index)
    return (device.type, 0)


def create_workers(devices: List[torch.device]) -> Tuple[List[InQueue], List[OutQueue]]:
    """Queues per entry of ``devices``; entries naming the same device share one thread and one queue pair."""
    pairs: Dict[Hashable, Tuple[InQueue, OutQueue]] = {}
    for device in devices:
        key = _device_key(device)
        if key not in pairs:
            pairs[key] = (Queue(), Queue())
            threading.Thread(target=worker, args=(*pairs[key], torch.device(device)), daemon=True).start()
    chosen = [pairs[_device_key(d)] for d in devices]
    return [p[0] for p in chosen], [p[1] for p in chosen]


def join_workers(in_queues: List[InQueue], out_queues: List[OutQueue]) -> None:
    """Stop the threads behind the queues and wait for their termination markers."""
    if sys.is_finalizing():
        return  # daemon threads do not survive interpreter shutdown; nothing to wait for
    for q in {id(q): q for q in in_queues}.values():
        q.put(None)
    for q in {id(q): q for q in out_queues}.values():
        try:
            while q.get(timeout=2.0) != (False, None):
                pass  # a stale result or exception record
        except Empty:
            pass  # the thread is gone already


@contextmanager
def spawn_workers(devices: List[torch.device]) -> Generator[Tuple[List[InQueue], List[OutQueue]], None, None]:
    queues = create_workers(devices)
    try:
        yield queues
    finally:
        join_workers(*queues)
