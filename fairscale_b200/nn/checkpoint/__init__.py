from .checkpoint_activations import (  # noqa: F401
    checkpoint_invocations,
    checkpoint_wrapper,
    disable_checkpointing,
    is_checkpointing,
    is_recomputing,
)
