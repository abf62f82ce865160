from .distributed import SlowMoBaseAlgorithm, SlowMoDistributedDataParallel  # noqa: F401
from .gossiper import PushPull, PushSum  # noqa: F401
from .graph_manager import (  # noqa: F401
    DynamicBipartiteExponentialGraph,
    DynamicBipartiteLinearGraph,
    DynamicDirectedExponentialGraph,
    DynamicDirectedLinearGraph,
    GraphManager,
    NPeerDynamicDirectedExponentialGraph,
    RingGraph,
)
from .mixing_manager import MixingManager, UniformMixing  # noqa: F401
from .utils import communicate  # noqa: F401
from .utils.cuda_metering import CudaEventRecorder  # noqa: F401
