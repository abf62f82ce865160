"""Optimizers and gradient scalers (mirrors fairscale/optim/__init__.py:12-22)."""
from .oss import OSS  # noqa: F401
from .adam import Adam, FusedAdam, Precision  # noqa: F401
