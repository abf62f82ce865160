"""Skip tensors as stage ports (this module takes the place of fairscale/nn/pipe/skip/portal.py).

The reference hides a skip tensor from autograd inside a ``Portal`` object and re-creates its graph edges with three
autograd functions (``PortalBlue``, ``PortalOrange``, ``PortalCopy``) and a reference-counted tensor life.  Here a skip
tensor that crosses partitions is an ordinary extra output of the stage that stashes it and an ordinary extra input of
the stage that pops it (:class:`SkipPort` names such a port), so the pipeline's regular machinery applies to it
unchanged: ``Copy`` / ``Wait`` move it between devices on the copy streams, ``Checkpoint`` / ``Recompute`` save and
replay it with the stage's other inputs, and its gradient flows back through the same nodes.  There are no portal
objects, hence no tensor-life counting and nothing to leak when a backward pass is skipped.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

from .namespace import Namespace

__all__: List[str] = []


@dataclass(frozen=True)
class SkipPort:
    """One routed skip tensor: stashed as ``(ns, name)`` in partition ``src``, popped in partition ``dst``."""

    ns: Optional[Namespace]
    name: str
    src: int
    dst: int
