"""Namespaces isolate skip-tensor names between module instances (parity: fairscale/nn/pipe/skip/namespace.py:29-63)."""

from __future__ import annotations

import abc
import uuid
from functools import total_ordering
from typing import Any

__all__ = ["Namespace"]


@total_ordering
class Namespace(metaclass=abc.ABCMeta):
    """A unique, hashable, orderable token; ``None`` is accepted wherever a namespace is (default namespace)."""

    __slots__ = ("id",)

    def __init__(self) -> None:
        self.id = uuid.uuid4()

    def __repr__(self) -> str:
        return f"<Namespace '{self.id}'>"

    def __hash__(self) -> int:
        return hash(self.id)

    def __lt__(self, other: Any) -> bool:  # ordering only serves deterministic sorting of layouts
        if isinstance(other, Namespace):
            return self.id < other.id
        return False

    def __eq__(self, other: Any) -> bool:
        if isinstance(other, Namespace):
            return self.id == other.id
        return False


Namespace.register(type(None))
