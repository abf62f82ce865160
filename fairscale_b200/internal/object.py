"""Pickle python objects into fixed-size uint8 tensors (parity: fairscale/internal/object.py:12-29)."""

from __future__ import annotations

import io
import pickle
from typing import Any

import torch


def pyobject_to_tensor(obj: Any, fixed_buffer_size: int = 0) -> torch.Tensor:
    """Serialise ``obj`` to a uint8 tensor; zero-pad to ``fixed_buffer_size`` when given."""
    payload = pickle.dumps(obj)
    assert fixed_buffer_size == 0 or len(payload) <= fixed_buffer_size
    size = max(len(payload), fixed_buffer_size)
    out = torch.zeros(size, dtype=torch.uint8)
    out[: len(payload)] = torch.frombuffer(bytearray(payload), dtype=torch.uint8)
    return out


def tensor_to_pyobject(tensor: torch.Tensor) -> Any:
    """Inverse of :func:`pyobject_to_tensor` (trailing zero padding is ignored by pickle)."""
    return pickle.load(io.BytesIO(tensor.cpu().numpy().tobytes()))
