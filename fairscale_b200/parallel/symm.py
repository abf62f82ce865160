"""Registry of NVLink symmetric-memory workspaces, one per process group.

A workspace owns peer-mapped staging buffers and signal pads for a group and exposes
the hand-written collectives.  The registry is empty until
:func:`fairscale_b200.parallel.nvlink.enable` is called on a multi-GPU NVLink box.

Workspaces are keyed by the group's member ranks (not by the Python object's identity, which a later group can
reuse once the first one has been collected).
"""

from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

_WORKSPACES: Dict[Tuple[int, ...], Any] = {}


def _key(group: Any) -> Tuple[int, ...]:
    import torch.distributed as dist

    try:
        if group is None or group is dist.group.WORLD:
            return tuple(range(dist.get_world_size()))
        return tuple(dist.get_process_group_ranks(group))
    except Exception:
        return (-1, id(group))


def register_workspace(group: Any, ws: Any) -> None:
    _WORKSPACES[_key(group)] = ws


def unregister_all() -> None:
    _WORKSPACES.clear()


def workspace_for(group: Any) -> Optional[Any]:
    """The usable workspace of ``group``; None if there is none or a kernel of it reported a failed wait."""
    if not _WORKSPACES:
        return None
    ws = _WORKSPACES.get(_key(group))
    if ws is not None and getattr(ws, "poisoned", False):
        return None
    return ws


def poison_all() -> None:
    """Mark every workspace unusable: called when a kernel gave up a bounded wait, which leaves the flags, counters
    and epochs of the in-kernel collectives in an unknown state.  Callers fall back to ``torch.distributed``."""
    for ws in _WORKSPACES.values():
        ws.poisoned = True


def heap_allocator(group: Any, tag: str) -> Optional[Any]:
    """An ``allocator(numel, dtype, device)`` for flat buckets that places them in the symmetric heap of ``group``'s
    workspace (so that peers can pull them directly), or None without a workspace.  Every call hands out fresh memory: a
    bucket that is rebuilt copies its members' values out of the old buffer, which therefore must not be recycled under
    it.  Every rank must allocate the same buckets in the same order (the heap hands out the same offsets on every rank);
    when the heap is full the bucket goes to ordinary device memory, on every rank alike since sizes are the same
    everywhere.  ``tag`` only labels the allocation for debugging."""
    ws = workspace_for(group)
    if ws is None:
        return None
    import torch

    def allocate(numel: int, dtype: "torch.dtype", device: "torch.device") -> "torch.Tensor":
        if torch.device(device) != ws.device or numel == 0:
            return torch.empty(numel, dtype=dtype, device=device)
        try:
            return ws.alloc_tensor((numel,), dtype)
        except MemoryError:
            return torch.empty(numel, dtype=dtype, device=device)

    return allocate
