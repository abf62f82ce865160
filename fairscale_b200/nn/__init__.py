"""Public neural-network API (mirrors fairscale/nn/__init__.py:10-20)."""
from .data_parallel import FullyShardedDataParallel, ShardedDataParallel  # noqa: F401
from .misc import FlattenParamsWrapper  # noqa: F401
from .wrap import auto_wrap, config_auto_wrap_policy, default_auto_wrap_policy, enable_wrap, wrap  # noqa: F401
