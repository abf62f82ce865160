"""Pipeline parallelism (mirrors fairscale/nn/pipe/__init__.py)."""
from .checkpoint import is_checkpointing, is_recomputing  # noqa: F401
from .pipe import Pipe  # noqa: F401

__all__ = ["Pipe", "is_checkpointing", "is_recomputing"]
