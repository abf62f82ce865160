from .flatten_params_wrapper import FlatParameter, FlattenParamsWrapper  # noqa: F401
from .param_bucket import GradBucket, ParamBucket  # noqa: F401
