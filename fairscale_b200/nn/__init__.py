"""Public neural-network API (mirrors fairscale/nn/__init__.py:10-24)."""
from .checkpoint import checkpoint_wrapper  # noqa: F401
from .data_parallel import FullyShardedDataParallel, ShardedDataParallel  # noqa: F401
from .misc import FlattenParamsWrapper  # noqa: F401
from .moe import MOELayer, Top2Gate  # noqa: F401
from .pipe import AsyncPipe, Pipe  # noqa: F401
from .pipe.rpc import PipeRPCWrapper  # noqa: F401
from .wrap import auto_wrap, config_auto_wrap_policy, default_auto_wrap_policy, enable_wrap, wrap  # noqa: F401

__all__ = [
    "checkpoint_wrapper", "FullyShardedDataParallel", "ShardedDataParallel", "FlattenParamsWrapper", "MOELayer", "Top2Gate",
    "Pipe", "AsyncPipe", "PipeRPCWrapper", "auto_wrap", "config_auto_wrap_policy", "default_auto_wrap_policy", "enable_wrap", "wrap",
]
