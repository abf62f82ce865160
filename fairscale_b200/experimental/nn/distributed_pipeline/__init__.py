from .graph import PipelineModulesGraph  # noqa: F401
from .loss import DistributedLoss  # noqa: F401
from .pipeline import DistributedPipeline  # noqa: F401
from .trace import make_graph  # noqa: F401

__all__ = ["PipelineModulesGraph", "DistributedLoss", "DistributedPipeline", "make_graph"]
