"""Registry of NVLink symmetric-memory workspaces, one per process group.

A workspace owns peer-mapped staging buffers and signal pads for a group and exposes
the hand-written collectives.  The registry is empty until
:func:`fairscale_b200.parallel.nvlink.enable` is called on a multi-GPU NVLink box.
"""

from __future__ import annotations

from typing import Any, Dict, Optional

_WORKSPACES: Dict[int, Any] = {}


def register_workspace(group: Any, ws: Any) -> None:
    _WORKSPACES[id(group)] = ws


def unregister_all() -> None:
    _WORKSPACES.clear()


def workspace_for(group: Any) -> Optional[Any]:
    if not _WORKSPACES:
        return None
    return _WORKSPACES.get(id(group))
