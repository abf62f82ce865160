from .mevo import BaselineSoftmaxNllLoss, MemoryEfficientVocabOutput  # noqa: F401
from .offload import OffloadModel  # noqa: F401
from .sync_batchnorm import SyncBatchNorm  # noqa: F401

__all__ = ["MemoryEfficientVocabOutput", "BaselineSoftmaxNllLoss", "OffloadModel", "SyncBatchNorm"]
