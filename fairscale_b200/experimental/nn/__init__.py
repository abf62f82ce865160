from .mevo import BaselineSoftmaxNllLoss  # noqa: F401
from .mevo import MemoryEfficientVocabOutput  # noqa: F401
from .mevo import MemoryEfficientVocabOutput as MEVO  # noqa: F401
from .offload import OffloadModel  # noqa: F401
from .sync_batchnorm import SyncBatchNorm  # noqa: F401

__all__ = ["MEVO", "MemoryEfficientVocabOutput", "BaselineSoftmaxNllLoss", "OffloadModel", "SyncBatchNorm"]
