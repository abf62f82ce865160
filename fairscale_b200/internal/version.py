"""Version parsing (parity: fairscale/internal/version.py:16-32)."""

from __future__ import annotations

import logging
import re
from typing import Tuple

import torch

__all__ = ["torch_version"]

_NUMERIC = re.compile(r"^(\d+)\.(\d+)\.(\d+)")


def torch_version(version: str = torch.__version__) -> Tuple[int, ...]:
    """``"2.11.0+cu128"`` → ``(2, 11, 0)``; unparsable strings → ``()`` with a warning."""
    m = _NUMERIC.match(version)
    if m is None:
        logging.warning(f"Pytorch pre-release version {version} - assuming intent to test it")
        return ()
    return tuple(int(g) for g in m.groups())
