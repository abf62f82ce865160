"""Namespaces keep equal skip names apart: ``stash("x")`` isolated in one namespace only meets the ``pop("x")`` isolated
in the same one.  A namespace is an opaque identity; two of them are equal only if they are the same object.
(fairscale/nn/pipe/skip/namespace.py:16-50 orders and hashes them through a uuid; identity gives the same behaviour.)
"""

from __future__ import annotations

import itertools
from typing import Any

__all__ = ["Namespace"]

_serial = itertools.count()


class Namespace:
    __slots__ = ("id",)

    def __init__(self) -> None:
        self.id = next(_serial)

    def __repr__(self) -> str:
        return f"<Namespace #{self.id}>"

    def __hash__(self) -> int:
        return hash(("fsb-skip-namespace", self.id))

    def __eq__(self, other: Any) -> bool:
        return isinstance(other, Namespace) and other.id == self.id

    # sortable, so that error messages and port orders are deterministic
    def __lt__(self, other: Any) -> bool:
        if not isinstance(other, Namespace):
            return NotImplemented
        return self.id < other.id
