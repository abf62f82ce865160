"""Pipeline schedules as data: which (micro-batch, stage) pairs run at which clock.

``FillDrain`` is GPipe's schedule: all forwards in a diagonal wave (stage ``j`` runs micro-batch ``k - j`` at clock
``k``), the backward replays it in reverse through autograd.  ``OneFOneB`` lists, for one stage of a multi-process
pipeline, the interleaved order of forward and backward micro-batches that bounds the number of live activations by
the pipeline depth instead of the number of micro-batches.  The single-process ``Pipe``, ``AsyncPipe`` and the
benchmark drivers all take their order of work from these objects.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator, List, Tuple

__all__ = ["FillDrain", "OneFOneB"]


@dataclass(frozen=True)
class FillDrain:
    """``m`` micro-batches through ``n`` stages in ``m + n - 1`` clocks."""

    m: int
    n: int

    def __len__(self) -> int:
        return self.m + self.n - 1 if self.m > 0 and self.n > 0 else 0

    def clock(self, k: int) -> List[Tuple[int, int]]:
        """``[(micro-batch, stage), ...]`` active at clock ``k``, earliest stage first."""
        first_stage = max(k - self.m + 1, 0)
        last_stage = min(k, self.n - 1)
        return [(k - j, j) for j in range(first_stage, last_stage + 1)]

    def __iter__(self) -> Iterator[List[Tuple[int, int]]]:
        return (self.clock(k) for k in range(len(self)))


@dataclass(frozen=True)
class OneFOneB:
    """Order of work of stage ``stage`` (0-based) of ``n`` for ``m`` micro-batches: warm-up forwards, then one forward
    and one backward alternately, then the remaining backwards."""

    m: int
    n: int
    stage: int

    def __iter__(self) -> Iterator[Tuple[str, int]]:
        warmup = min(self.n - self.stage - 1, self.m)
        fwd = bwd = 0
        for _ in range(warmup):
            yield ("forward", fwd)
            fwd += 1
        while fwd < self.m:
            yield ("forward", fwd)
            fwd += 1
            yield ("backward", bwd)
            bwd += 1
        while bwd < self.m:
            yield ("backward", bwd)
            bwd += 1

    def max_live_activations(self) -> int:
        return min(self.n - self.stage, self.m)
