"""Small parameter/gradient helpers (parity: fairscale/internal/params.py:14-76)."""

from __future__ import annotations

from collections import abc
from dataclasses import dataclass
from math import inf
from typing import Any, Callable, List, Optional, Union

import torch
import torch.distributed as dist


@dataclass
class Workhandle:
    """An async collective handle plus the callback to run once it completed."""

    handle: Any
    callback: Optional[Callable] = None


def get_global_rank(group: Any, rank: int) -> int:
    """Translate a group-local rank into a global rank."""
    if group is None or group is dist.group.WORLD:
        return rank
    return dist.get_global_rank(group, rank)


def recursive_copy_to_device(value: Any, non_blocking: bool, device: torch.device) -> Any:
    """Copy every tensor found in nested lists/tuples/mappings to ``device``."""
    if isinstance(value, torch.Tensor):
        return value.to(device, non_blocking=non_blocking)
    if isinstance(value, (list, tuple)):
        moved = [recursive_copy_to_device(v, non_blocking=non_blocking, device=device) for v in value]
        return moved if isinstance(value, list) else tuple(moved)
    if isinstance(value, abc.Mapping):
        return {k: recursive_copy_to_device(v, non_blocking=non_blocking, device=device) for k, v in value.items()}
    return value


def calc_grad_norm(parameters: Union[torch.Tensor, List[torch.nn.Parameter]], p: float) -> torch.Tensor:
    """p-norm of all ``.grad`` tensors viewed as one vector, accumulated in fp32."""
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]  # type: ignore[list-item]
    with_grad = [q for q in parameters if q.grad is not None]
    if not with_grad:
        return torch.tensor(0.0)
    p = float(p)
    if p == inf:
        return max(q.grad.detach().abs().max() for q in with_grad)  # type: ignore[union-attr,return-value]
    grads = [q.grad.detach() for q in with_grad]  # type: ignore[union-attr]
    if p == 2.0 and grads[0].is_cuda:
        from ..ops import multi_tensor

        if multi_tensor.supported(grads):  # one launch per dtype, result stays on the device
            return multi_tensor.l2_norm(grads).to(dtype=with_grad[0].dtype)
    per_param = torch.stack([torch.norm(q.grad.detach(), p, dtype=torch.float32) for q in with_grad])  # type: ignore[union-attr]
    return torch.norm(per_param, p).to(dtype=with_grad[0].dtype)
