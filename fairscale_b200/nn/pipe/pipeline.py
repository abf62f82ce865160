"""Executor of the single-process pipeline: runs micro-batches through the stages in fill-drain order.

Every stage owns a device, its compute stream (the device's current stream) and one copy stream per micro-batch.  For
each clock of the schedule the executor first *prepares* the active (micro-batch, stage) pairs - ties the micro-batch to
its predecessor so that backward replays them in reverse order, starts the device-to-device copies of the activations
and of routed skip tensors on the copy streams - and then *launches* them: makes the compute stream wait for the copies,
runs the stage (under ``Checkpoint`` for the micro-batches that are recomputed in backward) and collects the outputs.
Work of different stages overlaps because kernel launches and peer copies are asynchronous; optional helper threads
(``threads=True``, see ``worker.py``) only matter for stages dominated by host code that releases the GIL.

Skip connections: a skip tensor that crosses stages is an extra output of the stage that stashes it and an extra input
of the stage that pops it (``skip/layout.py``), so it needs no special handling in checkpointing or autograd.

Behaviour (clock order, copy streams per stage and micro-batch, ``chunk%d-part%d`` ranges, first exception re-raised
after the clock has drained) follows fairscale/nn/pipe/pipeline.py:56-276.
"""

from __future__ import annotations

import sys
from dataclasses import dataclass, field
from types import TracebackType
from typing import Callable, Iterable, List, Optional, Tuple, Type, Union

import torch
from torch import Tensor, nn
from torch.autograd.profiler import record_function

from .checkpoint import Checkpointing
from .copy import Copy, Wait
from .dependency import fork, join
from .microbatch import Batch
from .schedule import FillDrain
from .skip.layout import SkipKey, SkipLayout
from .skip.tracker import StageSkipTracker, use_skip_tracker
from .stream import AbstractStream, current_stream, use_device
from .worker import Task, create_workers, join_workers

__all__: List[str] = []

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]
ExcInfo = Tuple[Type[BaseException], BaseException, TracebackType]


def _grad_carriers(values: Iterable[Tensor]) -> Tensors:
    """Integer / bool tensors come out of an autograd function with ``requires_grad`` set; cut that off."""
    return tuple(v if v.is_floating_point() else v.detach() for v in values)


def depend(fork_from: Batch, join_to: Batch) -> None:
    """Order two micro-batches in backward: everything behind ``join_to`` finishes before ``fork_from`` continues."""
    fork_from[0], token = fork(fork_from[0])
    join_to[0] = join(join_to[0], token)


def copy(batch: Batch, prev_stream: AbstractStream, next_stream: AbstractStream) -> None:
    """Move the batch to the device of ``next_stream``; the copy runs on the two copy streams."""
    batch[:] = _grad_carriers(Copy.apply(prev_stream, next_stream, *batch))


def wait(batch: Batch, prev_stream: AbstractStream, next_stream: AbstractStream) -> None:
    """Make ``next_stream`` wait for what ``prev_stream`` has queued (in backward the other way round)."""
    batch[:] = _grad_carriers(Wait.apply(prev_stream, next_stream, *batch))


def clock_cycles(m: int, n: int) -> Iterable[List[Tuple[int, int]]]:
    """The fill-drain schedule as a sequence of clocks, each a list of ``(micro-batch, stage)``.

    m=3, n=3:  [(0,0)]  [(1,0),(0,1)]  [(2,0),(1,1),(0,2)]  [(2,1),(1,2)]  [(2,2)]
    """
    return iter(FillDrain(m, n))


@dataclass
class _Ports:
    """How the last call of a stage function packed its result: main outputs first, then exported skip tensors."""

    n_main: int = 0
    atomic: bool = True
    exported: List[SkipKey] = field(default_factory=list)
    absent: List[SkipKey] = field(default_factory=list)  # exported as None


class Pipeline:
    """Runs lists of micro-batches through the partitions.  ``threads=True`` hands the stage work to one helper thread
    per device instead of issuing everything from the calling thread."""

    def __init__(self, partitions: List[nn.Sequential], devices: List[torch.device], copy_streams: List[List[AbstractStream]],
                 skip_layout: SkipLayout, checkpoint_stop: int, threads: bool = False) -> None:
        self.partitions = partitions
        self.devices = devices
        self.copy_streams = copy_streams
        self.skip_layout = skip_layout
        self.checkpoint_stop = checkpoint_stop
        self._queues: Optional[Tuple[list, list]] = create_workers(devices) if threads else None

    def __del__(self) -> None:
        if getattr(self, "_queues", None) is not None:
            join_workers(*self._queues)  # type: ignore[misc]

    # ------------------------------------------------------------------ driver
    def run(self, batches: List[Batch]) -> None:
        """All micro-batches through all stages; ``batches`` ends up holding the outputs of the last stage."""
        trackers = [StageSkipTracker(self.skip_layout, b.index) for b in batches]
        for clock in FillDrain(len(batches), len(self.partitions)):
            self.fence(batches, clock, trackers)
            self.compute(batches, clock, trackers)

    # ------------------------------------------------------------------ phase 1: dependencies and copies
    def fence(self, batches: List[Batch], schedule: List[Tuple[int, int]], trackers: List[StageSkipTracker]) -> None:
        for i, j in schedule:
            if i > 0 and j > 0:
                depend(batches[i - 1], batches[i])  # stage j-1 replays micro-batch i before i-1 in backward
            arrival = self.copy_streams[j][i]
            for src, ns, name in self.skip_layout.copy_policy(j):
                trackers[i].copy(batches[i], self.copy_streams[src][i], arrival, ns, name)
            if j > 0:
                copy(batches[i], self.copy_streams[j - 1][i], arrival)

    # ------------------------------------------------------------------ phase 2: stage work
    def _stage_call(self, i: int, j: int, tracker: StageSkipTracker, carried: List[SkipKey], n_main: int, atomic: bool,
                    ports: _Ports) -> Callable[[TensorOrTensors], TensorOrTensors]:
        """The function a stage runs for one micro-batch, in the form checkpointing needs: tensors in, tensors out.
        Inputs: the micro-batch (``n_main`` tensors, or one if ``atomic``) followed by the skip tensors ``carried``."""
        partition = self.partitions[j]
        exports = self.skip_layout.exports(j)

        def call(packed: TensorOrTensors) -> TensorOrTensors:
            values = (packed,) if torch.is_tensor(packed) else tuple(packed)
            main: TensorOrTensors = values[0] if atomic else values[:n_main]
            tracker.inbox.update(zip(carried, values[n_main:]))
            with use_skip_tracker(tracker), record_function("chunk%d-part%d" % (i, j)):
                out = partition(main)
            out_values = (out,) if torch.is_tensor(out) else tuple(out)
            ports.n_main, ports.atomic = len(out_values), torch.is_tensor(out)
            ports.exported = [k for k in exports if tracker.outbox.get(k) is not None]
            ports.absent = [k for k in exports if tracker.outbox.get(k) is None]
            extra = tuple(tracker.outbox.pop(k) for k in ports.exported)
            for k in ports.absent:
                tracker.outbox.pop(k, None)
            if not extra:
                return out
            return out_values + extra

        return call

    def compute(self, batches: List[Batch], schedule: List[Tuple[int, int]], trackers: List[StageSkipTracker]) -> None:
        training = self.partitions[0].training
        checkpoint_stop = self.checkpoint_stop if training else 0  # evaluation keeps no graph: nothing to recompute
        streams = [current_stream(d) for d in self.devices]
        last = len(self.partitions) - 1
        launched: List[Tuple[int, int, Task, _Ports]] = []

        for i, j in schedule:
            batch, tracker = batches[i], trackers[i]
            if j > 0:
                wait(batch, self.copy_streams[j][i], streams[j])
            carried, skips = tracker.deliver(self.skip_layout.imports(j), self.copy_streams[j][i], streams[j])
            ports = _Ports()
            call = self._stage_call(i, j, tracker, carried, len(batch), batch.atomic, ports)
            packed = Batch(tuple(batch) + tuple(skips), batch.index) if skips else batch
            if i < checkpoint_stop:
                ckpt = Checkpointing(call, packed)
                task = Task(streams[j], compute=ckpt.checkpoint, finalize=ckpt.recompute)
            else:
                task = Task(streams[j], compute=lambda packed=packed, call=call: packed.call(call), finalize=None)  # type: ignore[misc]
            launched.append((i, j, task, ports))
            if self._queues is not None:
                self._queues[0][j].put(task)

        failure: Optional[ExcInfo] = None
        for i, j, task, ports in launched:
            if self._queues is not None:
                ok, payload = self._queues[1][j].get()  # always drained, so no thread is left holding a result
                if not ok:
                    failure = failure or payload
                    continue
                result: Batch = payload[1]
            else:
                if failure is not None:
                    continue
                try:
                    with use_device(self.devices[j]):
                        result = task.compute()
                except Exception:
                    failure = sys.exc_info()  # type: ignore[assignment]
                    continue
            if failure is not None:
                continue
            if j != last:
                wait(result, streams[j], self.copy_streams[j][i])  # the outgoing copies start after the stage's kernels
            with use_device(self.devices[j]):
                task.finalize(result)
            # unpack: exported skip tensors wait in transit on this device, the rest is the micro-batch
            values = tuple(result)
            for key, tensor in zip(ports.exported, values[ports.n_main:]):
                trackers[i].in_transit[key] = tensor
            for key in ports.absent:
                trackers[i].in_transit[key] = None
            batches[i] = Batch(values[0] if ports.atomic else values[: ports.n_main], result.index)

        if failure is not None:
            raise failure[0].with_traceback(failure[1], failure[2])
