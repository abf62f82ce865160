"""Empty placeholder tensors: they carry no data, only an edge of the autograd graph.

``get_phony(device, requires_grad=...)`` has the contract of fairscale/nn/pipe/phony.py:31-64 (one shared tensor per
device and flag, allocated outside any side stream so that no stream ever has to be recorded for it).
"""

from __future__ import annotations

import threading
from typing import Dict, List, Tuple

import torch
from torch import Tensor

__all__: List[str] = []

_lock = threading.Lock()
_cache: Dict[Tuple[str, int, bool], Tensor] = {}


def get_phony(device: torch.device, *, requires_grad: bool) -> Tensor:
    device = torch.device(device)
    key = (device.type, -1 if device.index is None else device.index, bool(requires_grad))
    hit = _cache.get(key)
    if hit is not None:
        return hit
    with _lock:
        if key not in _cache:
            if device.type == "cuda":
                # on the device's default stream: a tensor born there needs no record_stream bookkeeping
                with torch.cuda.stream(torch.cuda.default_stream(device)):
                    t = torch.empty(0, device=device, requires_grad=requires_grad)
            else:
                t = torch.empty(0, device=device, requires_grad=requires_grad)
            _cache[key] = t
        return _cache[key]
