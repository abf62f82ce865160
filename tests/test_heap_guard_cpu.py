"""Guard words of the bump-allocated heap, on a CPU tensor: guards are planted behind every window, an overrun is reported
with the window and the first byte it reached, underruns into the previous window's guard are reported against that window,
and restoring the guards separates one overrun from the next.  The workspace's allocator uses the same object when
``FSB200_HEAP_CANARY=1``; here a stand-in with the allocator's arithmetic checks the offsets and the off-by-default switch."""
import pytest
import torch

from fairscale_b200.parallel import heap_guard
from fairscale_b200.parallel.heap_guard import GUARD_BYTES, PATTERN, HeapGuards


class _Bump:
    """The allocator arithmetic of the NVLink workspace over a plain tensor."""

    def __init__(self, nbytes, guarded):
        self.heap = torch.zeros(nbytes, dtype=torch.uint8)
        self.bump = 0
        self.guards = HeapGuards(self.heap) if guarded else None

    def alloc(self, nbytes, align=256):
        off = (self.bump + align - 1) // align * align
        taken = nbytes if self.guards is None else self.guards.reserve(nbytes)
        if off + taken > self.heap.numel():
            raise MemoryError
        self.bump = off + taken
        if self.guards is not None:
            self.guards.plant(off, nbytes, label=f"w{len(self.guards.windows)}")
        return self.heap[off: off + nbytes]


def test_guards_sit_behind_every_window_and_report_overruns():
    heap = _Bump(8192, guarded=True)
    a, b, c = heap.alloc(100), heap.alloc(512), heap.alloc(256)
    offsets = [w.data_ptr() - heap.heap.data_ptr() for w in (a, b, c)]
    assert offsets == [0, 512, 1280]  # 100 + 256 guard -> next multiple of 256; 512 + 256; ...
    assert all(o % 256 == 0 for o in offsets)
    assert heap.guards.corrupted() == []
    for w in (a, b, c):
        w.fill_(7)  # writing inside the windows never trips a guard
    assert heap.guards.corrupted() == [] and int(heap.heap[100]) == PATTERN and int(heap.heap[100 + GUARD_BYTES - 1]) == PATTERN

    heap.heap[512 + 512 + 3: 512 + 512 + 9].fill_(1)  # six bytes past the second window, starting at the fourth
    report = heap.guards.corrupted()
    assert len(report) == 1 and report[0].startswith("w1:") and "first overwritten byte 3 " in report[0] and "6 of 256" in report[0]
    heap.guards.replant()
    assert heap.guards.corrupted() == []
    heap.heap[1279] = 0  # the byte just before the third window: the end of the second window's guard
    assert heap.guards.corrupted()[0].startswith("w1:") and "byte 255 " in heap.guards.corrupted()[0]
    heap.heap[100] = PATTERN ^ 0xFF
    assert [r.split(":")[0] for r in heap.guards.corrupted()] == ["w0", "w1"]


def test_unguarded_allocation_is_back_to_back_and_exhaustion_counts_the_guards():
    plain = _Bump(1024, guarded=False)
    first, second = plain.alloc(256), plain.alloc(256)
    assert second.data_ptr() - first.data_ptr() == 256
    plain.alloc(512)
    guarded = _Bump(1024, guarded=True)
    guarded.alloc(256)
    guarded.alloc(256)
    with pytest.raises(MemoryError):
        guarded.alloc(256)  # would fit without guards
    with pytest.raises(AssertionError):
        HeapGuards(torch.zeros(16, dtype=torch.uint8)).plant(0, 16)  # no room for the guard itself


def test_switch_is_off_by_default(monkeypatch):
    monkeypatch.delenv("FSB200_HEAP_CANARY", raising=False)
    assert not heap_guard.enabled()
    monkeypatch.setenv("FSB200_HEAP_CANARY", "1")
    assert heap_guard.enabled()
    with pytest.raises(AssertionError):
        HeapGuards(torch.zeros(4, 4, dtype=torch.uint8))
