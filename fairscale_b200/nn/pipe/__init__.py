"""Pipeline parallelism (mirrors fairscale/nn/pipe/__init__.py)."""
from .checkpoint import is_checkpointing, is_recomputing  # noqa: F401
from .async_pipe import AsyncPipe  # noqa: F401
from .async_pipeline import AsyncPipeline  # noqa: F401
from .async_schedule import AsyncEventLoop, Invocation, Location, ModuleWrapper  # noqa: F401
from .pipe import Pipe  # noqa: F401
from .rpc import PipeRPCWrapper  # noqa: F401
from .types import LazyModule  # noqa: F401

__all__ = ["Pipe", "AsyncPipe", "AsyncPipeline", "AsyncEventLoop", "LazyModule", "PipeRPCWrapper", "is_checkpointing", "is_recomputing"]
