"""Zero-cost placeholder tensors used to draw autograd edges (parity: fairscale/nn/pipe/phony.py:31-64)."""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch
from torch import Tensor

from .stream import default_stream, use_stream

__all__: List[str] = []

_phonies: Dict[Tuple[torch.device, bool], Tensor] = {}


def get_phony(device: torch.device, *, requires_grad: bool) -> Tensor:
    """A cached empty tensor on ``device``; it carries no data, only graph structure."""
    key = (device, requires_grad)
    phony = _phonies.get(key)
    if phony is None:
        with use_stream(default_stream(device)):
            phony = torch.empty(0, device=device, requires_grad=requires_grad)
        _phonies[key] = phony
    return phony
