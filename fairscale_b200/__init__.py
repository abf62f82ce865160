"""fairscale_b200: sharded / pipelined / expert / tensor-parallel training for NVIDIA B200 (sm_100a).

Sub-packages: ``nn`` (FSDP, ShardedDDP, Pipe, MoE, model_parallel, checkpoint, wrap), ``optim`` (OSS, fused Adam,
AdaScale, scalers), ``ops`` (tcgen05 / TMA kernels and their autograd functions), ``parallel`` (NVLink collectives
and the communication front-end), ``models``, ``experimental``, ``fair_dev`` (test support), ``utils``.
Like the reference (fairscale/__init__.py:16-20) only ``nn`` is imported eagerly.
"""

from . import nn  # noqa: F401
from .version import __version_tuple__

__version__ = ".".join(str(x) for x in __version_tuple__)
__all__ = ["nn", "__version__"]
