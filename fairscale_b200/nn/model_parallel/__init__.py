"""Tensor (model) parallelism (mirrors fairscale/nn/model_parallel/__init__.py)."""
from .cross_entropy import vocab_parallel_cross_entropy  # noqa: F401
from .initialize import (  # noqa: F401
    destroy_model_parallel,
    get_context_parallel_group,
    get_context_parallel_rank,
    get_context_parallel_ranks,
    get_context_parallel_world_size,
    get_data_parallel_group,
    get_data_parallel_rank,
    get_data_parallel_ranks,
    get_data_parallel_world_size,
    get_model_parallel_group,
    get_model_parallel_rank,
    get_model_parallel_src_rank,
    get_model_parallel_world_size,
    get_pipeline_parallel_group,
    get_pipeline_parallel_ranks,
    initialize_model_parallel,
    model_parallel_is_initialized,
)
from .layers import ColumnParallelLinear, ParallelEmbedding, RowParallelLinear, VocabParallelEmbedding  # noqa: F401
from .mappings import (  # noqa: F401
    copy_to_model_parallel_region,
    gather_from_model_parallel_region,
    reduce_from_model_parallel_region,
    scatter_to_model_parallel_region,
)
from .random import checkpoint, get_cuda_rng_tracker, model_parallel_cuda_manual_seed  # noqa: F401
