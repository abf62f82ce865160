"""Multi-tensor reductions and scaling in one launch per dtype (gradient norm, clipping, AMP unscale).

The reference computes the global gradient norm as a Python loop of ``torch.norm`` calls plus a ``stack``
(fairscale/internal/params.py:42-63) and unscales gradients through torch's foreach kernels
(fairscale/optim/grad_scaler.py:164-230).  Here every tensor of one dtype goes through a single kernel driven
by a pointer table in device memory, and the results (sum of squares, found-inf flag) stay on the device.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _bind

_TABLES: "OrderedDict[Tuple, Tuple[torch.Tensor, int]]" = OrderedDict()
_TABLE_CACHE = 128


def _table(tensors: Sequence[torch.Tensor]) -> Tuple[torch.Tensor, int]:
    """Device table of (ptr, numel, chunk_start, 0) rows for ``tensors``; cached because FSDP / OSS keep their
    gradient storage at fixed addresses from step to step."""
    chunk = _bind.fn("fsb_adam_chunk_size")()
    key = (tensors[0].device, tuple((t.data_ptr(), t.numel()) for t in tensors))
    hit = _TABLES.get(key)
    if hit is not None:
        _TABLES.move_to_end(key)
        return hit
    rows, start = [], 0
    for t in tensors:
        rows.append((t.data_ptr(), t.numel(), start, 0))
        start += (t.numel() + chunk - 1) // chunk
    table = torch.tensor(rows, dtype=torch.int64).to(tensors[0].device)
    _TABLES[key] = (table, start)
    if len(_TABLES) > _TABLE_CACHE:
        _TABLES.popitem(last=False)
    return table, start


def _by_dtype(tensors: Sequence[torch.Tensor]) -> Dict[torch.dtype, List[torch.Tensor]]:
    groups: Dict[torch.dtype, List[torch.Tensor]] = {}
    for t in tensors:
        if t.numel() == 0:
            continue
        assert t.is_contiguous(), "multi-tensor ops need contiguous tensors"
        groups.setdefault(t.dtype, []).append(t)
    return groups


def supported(tensors: Sequence[torch.Tensor]) -> bool:
    return len(tensors) > 0 and _bind.use_native(*tensors) and all(
        t.dtype in (torch.float32, torch.float16, torch.bfloat16) and t.is_contiguous() for t in tensors
    ) and len({t.device for t in tensors}) == 1


def sumsq(tensors: Sequence[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 one-element device tensor holding the sum of squares over all ``tensors``."""
    if not supported(tensors):
        acc = sum((t.float().pow(2).sum() for t in tensors), torch.zeros((), dtype=torch.float32, device=tensors[0].device if tensors else "cpu"))
        return acc.reshape(1) if out is None else out.copy_(acc.reshape(1))
    dev = tensors[0].device
    out = torch.zeros(1, dtype=torch.float32, device=dev) if out is None else out.zero_()
    for dt, group in _by_dtype(tensors).items():
        table, chunks = _table(group)
        _bind.call("fsb_multi_tensor_sumsq", table.data_ptr(), len(group), chunks, _bind.dtype_code(dt), out.data_ptr(), _bind.stream_ptr(dev))
    return out


def scale_(tensors: Sequence[torch.Tensor], scale: torch.Tensor, found_inf: Optional[torch.Tensor] = None) -> None:
    """``t *= scale`` for every tensor (``scale``: fp32 one-element tensor on the same device); when ``found_inf``
    (int32 one-element device tensor) is given it is set to 1 if any product is not finite."""
    if not tensors:
        return
    if not supported(tensors):
        for t in tensors:
            t.mul_(scale.to(t.device, t.dtype if t.is_floating_point() else torch.float32))
            if found_inf is not None and not bool(torch.isfinite(t).all()):
                found_inf.fill_(1)
        return
    dev = tensors[0].device
    assert scale.dtype == torch.float32 and scale.device == dev
    assert found_inf is None or (found_inf.dtype == torch.int32 and found_inf.device == dev)
    for dt, group in _by_dtype(tensors).items():
        table, chunks = _table(group)
        _bind.call("fsb_multi_tensor_scale", table.data_ptr(), len(group), chunks, _bind.dtype_code(dt), scale.data_ptr(),
                   None if found_inf is None else found_inf.data_ptr(), _bind.stream_ptr(dev))


def l2_norm(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    return sumsq(tensors).sqrt_().reshape(())
