"""Guard words between the windows of a bump-allocated heap (a race / overrun check for debugging).

The symmetric NVLink heap hands out windows back to back, and every peer can write into every window: a kernel that runs a
few bytes past its window corrupts a neighbour silently.  With ``FSB200_HEAP_CANARY=1`` the workspace leaves a guard of
``GUARD_BYTES`` bytes filled with ``PATTERN`` behind every window; :meth:`HeapGuards.corrupted` reads the guards back and names
the windows whose guard changed (:meth:`NvlinkWorkspace.check_canaries` raises with that list; call it between steps, it
synchronises the device).  Off by default: the guards cost heap space and the check a device synchronisation.

The class only needs a flat ``uint8`` tensor, so it is exercised on CPU tensors by the tests.
"""

from __future__ import annotations

import os
from typing import List, Tuple

import torch

GUARD_BYTES = 256
PATTERN = 0xA5


def enabled() -> bool:
    return os.environ.get("FSB200_HEAP_CANARY", "0") == "1"


class HeapGuards:
    """Book-keeping of the guards of one heap (``heap``: flat uint8 tensor that the caller allocates windows from)."""

    def __init__(self, heap: torch.Tensor, guard_bytes: int = GUARD_BYTES, pattern: int = PATTERN) -> None:
        assert heap.dtype == torch.uint8 and heap.dim() == 1
        self.heap = heap
        self.guard_bytes = guard_bytes
        self.pattern = pattern
        self.windows: List[Tuple[int, int, str]] = []  # (offset, bytes, label) of every guarded window

    def reserve(self, nbytes: int) -> int:
        """Bytes to take from the heap for a window of ``nbytes``: the window plus its guard."""
        return nbytes + self.guard_bytes

    def plant(self, offset: int, nbytes: int, label: str = "") -> None:
        """Fill the guard behind the window ``[offset, offset + nbytes)``; the caller reserved :meth:`reserve` bytes there."""
        end = offset + nbytes
        assert end + self.guard_bytes <= self.heap.numel(), "guard does not fit the heap"
        self.heap[end : end + self.guard_bytes].fill_(self.pattern)
        self.windows.append((offset, nbytes, label or f"window@{offset}"))

    def corrupted(self) -> List[str]:
        """Labels of the windows whose guard no longer holds the pattern, each with the offset of the first changed byte
        relative to the end of the window (one device-to-host read for all guards)."""
        if not self.windows:
            return []
        guards = torch.stack([self.heap[off + n : off + n + self.guard_bytes] for off, n, _ in self.windows])
        wrong = (guards != self.pattern).cpu()
        out = []
        for row, (_, _, label) in zip(wrong, self.windows):
            if bool(row.any()):
                out.append(f"{label}: first overwritten byte {int(row.nonzero()[0])} past the window, {int(row.sum())} of {self.guard_bytes} changed")
        return out

    def replant(self) -> None:
        """Restore every guard (after a report, to catch the next overrun separately)."""
        for off, n, _ in self.windows:
            self.heap[off + n : off + n + self.guard_bytes].fill_(self.pattern)
