"""Contiguous partition of a sequence into k blocks minimising the largest block sum.

Same contract as fairscale/nn/pipe/balance/blockpartition.py:30-108 (``solve(sequence, partitions)`` returns the
blocks); implemented as a binary search on the bottleneck value with a greedy feasibility check, followed by a
left-to-right fill that never leaves a later block empty.
"""

from __future__ import annotations

from typing import List

__all__ = ["solve"]


def _blocks_needed(seq: List[int], cap: float) -> int:
    blocks, cur = 1, 0.0
    for x in seq:
        if cur + x > cap and cur > 0:
            blocks += 1
            cur = 0.0
        cur += x
    return blocks


def solve(sequence: List[int], partitions: int = 1) -> List[List[int]]:
    if partitions < 1:
        raise ValueError(f"partitions must be a positive integer ({partitions} < 1)")
    n = len(sequence)
    if n < partitions:
        raise ValueError(f"sequence is shorter than intended partitions ({n} < {partitions})")
    lo, hi = float(max(sequence)), float(sum(sequence))
    # smallest bottleneck for which `partitions` blocks suffice (costs are integers or profiled floats)
    for _ in range(64):
        mid = (lo + hi) / 2
        if _blocks_needed(sequence, mid) <= partitions:
            hi = mid
        else:
            lo = mid
    cap = hi
    out: List[List[int]] = []
    cur: List[int] = []
    cur_sum = 0.0
    for idx, x in enumerate(sequence):
        remaining_items = n - idx
        remaining_blocks = partitions - len(out)
        must_close = cur and remaining_items == remaining_blocks - 1 + 0  # keep one item for each later block
        if cur and (cur_sum + x > cap * (1 + 1e-12) or remaining_items < remaining_blocks or must_close) and len(out) < partitions - 1:
            out.append(cur)
            cur, cur_sum = [], 0.0
        cur.append(x)
        cur_sum += x
    out.append(cur)
    while len(out) < partitions:  # split trailing blocks if the greedy pass used fewer than allowed
        big = max(range(len(out)), key=lambda i: len(out[i]))
        blk = out[big]
        if len(blk) < 2:
            break
        out[big : big + 1] = [blk[: len(blk) // 2], blk[len(blk) // 2 :]]
    return out
