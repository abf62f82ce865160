"""Pipeline parallelism (mirrors fairscale/nn/pipe/__init__.py)."""
from .checkpoint import is_checkpointing, is_recomputing  # noqa: F401
from .async_pipe import AsyncPipe  # noqa: F401
from .pipe import Pipe  # noqa: F401
from .types import LazyModule  # noqa: F401

__all__ = ["Pipe", "AsyncPipe", "LazyModule", "is_checkpointing", "is_recomputing"]
