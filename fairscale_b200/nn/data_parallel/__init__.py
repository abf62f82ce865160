from .sharded_ddp import ShardedDataParallel  # noqa: F401
