from .fully_sharded_data_parallel import (  # noqa: F401
    FullyShardedDataParallel,
    TrainingState,
    auto_wrap_bn,
    get_fsdp_instances,
    no_pre_load_state_dict_hook,
)
from .sharded_ddp import ShardedDataParallel  # noqa: F401
