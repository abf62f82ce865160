from .flatten_params_wrapper import FlatParameter, FlattenParamsWrapper  # noqa: F401
from .param_bucket import GradBucket, ParamBucket  # noqa: F401


def __getattr__(name: str):  # the reference re-exports checkpoint_wrapper here for backward compatibility
    if name == "checkpoint_wrapper":
        from ..checkpoint import checkpoint_wrapper

        return checkpoint_wrapper
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
