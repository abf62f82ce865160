"""Tensor (model) parallelism: process-group grid, the four region mappings, the parallel layers, the loss on vocabulary
shards and the random-number streams.  The public names are those of fairscale/nn/model_parallel/__init__.py; each
sub-module lists its own in ``__all__``."""

from . import cross_entropy, initialize, layers, mappings, random  # noqa: F401
from .cross_entropy import *  # noqa: F401,F403
from .initialize import *  # noqa: F401,F403
from .layers import *  # noqa: F401,F403
from .mappings import *  # noqa: F401,F403
from .random import *  # noqa: F401,F403

__all__ = cross_entropy.__all__ + initialize.__all__ + layers.__all__ + mappings.__all__ + random.__all__
