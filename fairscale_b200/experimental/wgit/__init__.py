"""wgit ("weigit"): version control for model weights with de-duplicated, optionally sparsified storage."""

from .repo import Repo, RepoStatus  # noqa: F401
from .sha1_store import SHA1_Store  # noqa: F401
from .signal_sparsity import Algo, SignalSparsity, random_sparse_mask  # noqa: F401
from .signal_sparsity_profiling import EnergyConcentrationProfile  # noqa: F401
from .version import __version_tuple__  # noqa: F401

__version__ = ".".join(str(x) for x in __version_tuple__)
