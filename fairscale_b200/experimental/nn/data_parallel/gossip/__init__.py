"""Gossip-based data parallelism: the SlowMo wrapper, the gossipers it drives, the communication graphs they walk and the
mixing rule.  Everything a user names lives one level down; this module gathers it (same public names as
fairscale/experimental/nn/data_parallel/gossip/__init__.py)."""

from . import distributed as _distributed
from . import gossiper as _gossiper
from . import graph_manager as _graphs
from . import mixing_manager as _mixing
from .utils import communicate  # noqa: F401
from .utils.cuda_metering import CudaEventRecorder  # noqa: F401

_EXPORTS = {
    _distributed: ("SlowMoBaseAlgorithm", "SlowMoDistributedDataParallel"),
    _gossiper: ("PushPull", "PushSum"),
    _graphs: ("GraphManager", "RingGraph", "DynamicDirectedExponentialGraph", "NPeerDynamicDirectedExponentialGraph",
              "DynamicBipartiteExponentialGraph", "DynamicDirectedLinearGraph", "DynamicBipartiteLinearGraph"),
    _mixing: ("MixingManager", "UniformMixing"),
}
for _module, _names in _EXPORTS.items():
    for _name in _names:
        globals()[_name] = getattr(_module, _name)

__all__ = [n for names in _EXPORTS.values() for n in names] + ["communicate", "CudaEventRecorder"]
