"""Small parameter/gradient helpers (parity: fairscale/internal/params.py:14-76)."""

from __future__ import annotations

import math
from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any, Callable, List, Optional, Union

import torch
import torch.distributed as dist

__all__ = ["Workhandle", "get_global_rank", "recursive_copy_to_device", "calc_grad_norm"]


@dataclass
class Workhandle:
    """What an asynchronous collective returned, and what to run when it is done."""

    handle: Any
    callback: Optional[Callable] = None


def get_global_rank(group: Any, rank: int) -> int:
    """``rank`` counted inside ``group`` -> the same process counted in the default group."""
    in_world = group is None or group is dist.group.WORLD
    return rank if in_world else dist.get_global_rank(group, rank)


def recursive_copy_to_device(value: Any, non_blocking: bool, device: torch.device) -> Any:
    """``value`` with every tensor inside it (lists, tuples and mappings are walked) moved to ``device``; anything else is
    returned as it is.  Mappings come back as plain dicts."""

    def walk(node: Any) -> Any:
        if torch.is_tensor(node):
            return node.to(device, non_blocking=non_blocking)
        if isinstance(node, Mapping):
            return {key: walk(item) for key, item in node.items()}
        if isinstance(node, tuple):
            return tuple(walk(item) for item in node)
        if isinstance(node, list):
            return [walk(item) for item in node]
        return node

    return walk(value)


def calc_grad_norm(parameters: Union[torch.Tensor, List[torch.nn.Parameter]], p: float) -> torch.Tensor:
    """The ``p``-norm of the gradients of ``parameters`` taken as one long vector.  Parameters without a gradient do not count;
    with none left the norm is 0.  Sums run in fp32 and the result has the dtype of the first parameter that counts."""
    owners = [parameters] if torch.is_tensor(parameters) else list(parameters)
    grads = [owner.grad.detach() for owner in owners if owner.grad is not None]
    if len(grads) == 0:
        return torch.tensor(0.0)
    out_dtype = next(owner.dtype for owner in owners if owner.grad is not None)
    order = float(p)
    if order == math.inf:
        return max(g.abs().max() for g in grads)  # type: ignore[return-value]
    if order == 2.0 and grads[0].is_cuda:
        from ..ops import multi_tensor

        if multi_tensor.supported(grads):  # one launch per dtype, result stays on the device
            return multi_tensor.l2_norm(grads).to(dtype=out_dtype)
    partial = torch.stack([torch.norm(g, order, dtype=torch.float32) for g in grads])
    return torch.norm(partial, order).to(dtype=out_dtype)
