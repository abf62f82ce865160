"""Optimizers, optimizer wrappers and loss scalers."""

from .adam import Adam, FusedAdam, Precision  # noqa: F401
from .adascale import AdaScale, AdaScaleWrapper  # noqa: F401
from .grad_scaler import GradScaler, ShardedGradScaler  # noqa: F401
from .layerwise_gradient_scaler import LayerwiseGradientScaler  # noqa: F401
from .oss import OSS  # noqa: F401

__all__ = ["Adam", "FusedAdam", "Precision", "AdaScale", "AdaScaleWrapper", "GradScaler", "ShardedGradScaler",
           "LayerwiseGradientScaler", "OSS"]
