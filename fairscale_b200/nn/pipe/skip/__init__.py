"""Skip connections for pipelines (mirrors fairscale/nn/pipe/skip/__init__.py)."""
from .namespace import Namespace  # noqa: F401
from .skippable import pop, skippable, stash, verify_skippables  # noqa: F401

__all__ = ["skippable", "stash", "pop", "verify_skippables", "Namespace"]
