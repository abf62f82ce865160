"""GPipe clock-cycle scheduler for a single-process, multi-device pipeline.

Parity: fairscale/nn/pipe/pipeline.py:56-276.  At clock ``k`` stage ``j`` processes micro-batch ``k - j``.
Per clock: (1) *fence* — order micro-batch backward with fork/join, move skip tensors and the activations to
the next device on per-(stage, micro-batch) copy streams (NVLink peer copies on one box); (2) *compute* — hand
one task per active stage to that stage's worker thread, collect results, make copy streams wait for compute,
attach early recomputation.
"""

from __future__ import annotations

from queue import Queue
from types import TracebackType
from typing import TYPE_CHECKING, Iterable, List, Optional, Tuple, Type, Union, cast

import torch
from torch import Tensor, nn
from torch.autograd.profiler import record_function

from .checkpoint import Checkpointing
from .copy import Copy, Wait
from .dependency import fork, join
from .microbatch import Batch
from .skip.layout import SkipLayout
from .skip.tracker import SkipTrackerThroughPotals, use_skip_tracker
from .stream import AbstractStream, current_stream, use_device
from .worker import Task, create_workers, join_workers

__all__: List[str] = []

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]
ExcInfo = Tuple[Type[BaseException], BaseException, TracebackType]


def depend(fork_from: Batch, join_to: Batch) -> None:
    """Backward of ``join_to`` must finish before backward of ``fork_from`` proceeds."""
    fork_from[0], phony = fork(fork_from[0])
    join_to[0] = join(join_to[0], phony)


def copy(batch: Batch, prev_stream: AbstractStream, next_stream: AbstractStream) -> None:
    batch[:] = Copy.apply(prev_stream, next_stream, *batch)
    batch[:] = tuple(x if x.is_floating_point() else x.detach() for x in batch)  # only floats carry gradients


def wait(batch: Batch, prev_stream: AbstractStream, next_stream: AbstractStream) -> None:
    batch[:] = Wait.apply(prev_stream, next_stream, *batch)
    batch[:] = tuple(x if x.is_floating_point() else x.detach() for x in batch)


def clock_cycles(m: int, n: int) -> Iterable[List[Tuple[int, int]]]:
    """Schedules ``[(micro-batch i, stage j), ...]`` for each of the ``m + n - 1`` clocks.

    m=3, n=3:  k=0 [(0,0)]  k=1 [(1,0),(0,1)]  k=2 [(2,0),(1,1),(0,2)]  k=3 [(2,1),(1,2)]  k=4 [(2,2)]
    """
    for k in range(m + n - 1):
        yield [(k - j, j) for j in range(max(1 + k - m, 0), min(1 + k, n))]


class Pipeline:
    def __init__(self, partitions: List[nn.Sequential], devices: List[torch.device], copy_streams: List[List[AbstractStream]],
                 skip_layout: SkipLayout, checkpoint_stop: int) -> None:
        self.partitions = partitions
        self.devices = devices
        self.copy_streams = copy_streams
        self.skip_layout = skip_layout
        self.checkpoint_stop = checkpoint_stop
        self.in_queues, self.out_queues = create_workers(devices)

    def __del__(self) -> None:
        join_workers(self.in_queues, self.out_queues)

    def run(self, batches: List[Batch]) -> None:
        """Run all micro-batches through all stages; ``batches`` is updated in place."""
        m, n = len(batches), len(self.partitions)
        trackers = [SkipTrackerThroughPotals(self.skip_layout, i) for i in range(m)]
        for schedule in clock_cycles(m, n):
            self.fence(batches, schedule, trackers)
            self.compute(batches, schedule, trackers)

    def fence(self, batches: List[Batch], schedule: List[Tuple[int, int]], trackers: List[SkipTrackerThroughPotals]) -> None:
        for i, j in schedule:
            if i != 0 and j != 0:
                depend(batches[i - 1], batches[i])  # micro-batch i-1 finishes its backward on stage j after micro-batch i
            next_stream = self.copy_streams[j][i]
            for prev_j, ns, name in self.skip_layout.copy_policy(j):
                trackers[i].copy(batches[i], self.copy_streams[prev_j][i], next_stream, ns, name)
            if j != 0:
                copy(batches[i], self.copy_streams[j - 1][i], next_stream)

    def compute(self, batches: List[Batch], schedule: List[Tuple[int, int]], trackers: List[SkipTrackerThroughPotals]) -> None:
        n = len(self.partitions)
        checkpoint_stop = self.checkpoint_stop if self.partitions[0].training else 0  # no checkpointing in eval
        streams = [current_stream(d) for d in self.devices]
        exc_info: Optional[ExcInfo] = None

        for i, j in schedule:
            batch, partition = batches[i], self.partitions[j]
            if j != 0:
                wait(batch, self.copy_streams[j][i], streams[j])  # compute waits for the incoming copy
            if i < checkpoint_stop:

                def function(input: TensorOrTensors, partition: nn.Sequential = partition,
                             tracker: SkipTrackerThroughPotals = trackers[i], chunk: int = i, part: int = j) -> TensorOrTensors:
                    with use_skip_tracker(tracker), record_function("chunk%d-part%d" % (chunk, part)):
                        return partition(input)

                chk = Checkpointing(function, batch)
                task = Task(streams[j], compute=chk.checkpoint, finalize=chk.recompute)
                del function, chk
            else:

                def compute(batch: Batch = batch, partition: nn.Sequential = partition,
                            tracker: SkipTrackerThroughPotals = trackers[i], chunk: int = i, part: int = j) -> Batch:
                    with use_skip_tracker(tracker), record_function("chunk%d-part%d" % (chunk, part)):
                        return batch.call(partition)

                task = Task(streams[j], compute=compute, finalize=None)
                del compute
            self.in_queues[j].put(task)

        for i, j in schedule:
            ok, payload = self.out_queues[j].get()
            if exc_info is not None:
                continue  # keep draining so no worker is left with a pending result
            if not ok:
                exc_info = cast(ExcInfo, payload)
                continue
            task, batch = cast(Tuple[Task, Batch], payload)
            if j != n - 1:
                wait(batch, streams[j], self.copy_streams[j][i])  # the outgoing copy waits for compute
            with use_device(self.devices[j]):
                task.finalize(batch)
            batches[i] = batch

        if exc_info is not None:
            raise exc_info[0].with_traceback(exc_info[1], exc_info[2])
