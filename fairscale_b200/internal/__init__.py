"""Internal helpers; not part of the public API (mirrors fairscale/internal)."""
from .version import torch_version  # noqa: F401
