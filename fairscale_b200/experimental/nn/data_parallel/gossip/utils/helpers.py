"""Flatten / communicate / unflatten helpers (parity: fairscale/experimental/nn/data_parallel/gossip/utils/helpers.py:18-157)."""

from __future__ import annotations

import collections
import logging
import sys
from typing import Any, Callable, Dict, List, MutableMapping, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def flatten_tensors(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    """One contiguous 1-D tensor holding all ``tensors`` (same dtype) back to back."""
    if len(tensors) == 1:
        return tensors[0].reshape(-1).clone()
    return torch.cat([t.reshape(-1) for t in tensors], dim=0)


def unflatten_tensors(flat: torch.Tensor, tensors: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    """Views of ``flat`` shaped like ``tensors``."""
    out, off = [], 0
    for t in tensors:
        out.append(flat[off : off + t.numel()].view_as(t))
        off += t.numel()
    return out


def group_by_dtype(tensors: Sequence[torch.Tensor]) -> Dict[torch.dtype, List[torch.Tensor]]:
    groups: Dict[torch.dtype, List[torch.Tensor]] = collections.defaultdict(list)
    for t in tensors:
        groups[t.dtype].append(t)
    return groups


def communicate(tensors: Sequence[torch.Tensor], communication_op: Callable[..., Any], logger: Optional[logging.Logger] = None) -> None:
    """Run ``communication_op(tensor=flat)`` once per dtype over the flattened tensors and copy the result back."""
    with torch.no_grad():
        for dt, group in group_by_dtype(tensors).items():
            flat = flatten_tensors(group)
            if logger is not None:
                logger.debug("communicating %d elements of %s", flat.numel(), dt)
            communication_op(tensor=flat)
            torch._foreach_copy_(list(group), unflatten_tensors(flat, group))


def create_process_group(ranks: List[int]) -> Any:
    """New process group over ``ranks`` (collective over the whole world); warmed up with one all-reduce on its members."""
    group = dist.new_group(ranks)
    if dist.get_rank() in ranks:
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
        dist.all_reduce(torch.ones(1, device=dev), group=group)
    return group


class MultiProcessAdapter(logging.LoggerAdapter):
    """Prefix every record with the process rank."""

    def process(self, msg: str, kwargs: Any) -> Tuple[str, MutableMapping[str, Any]]:
        return f"process: {self.extra['process_num']} {msg}", kwargs  # type: ignore[index]


def make_logger(rank: int, verbose: bool = True) -> logging.Logger:
    logger = logging.getLogger(__name__ + f".rank{rank}")
    if not logger.handlers:
        h = logging.StreamHandler(stream=sys.stdout)
        h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s: %(message)s"))
        logger.addHandler(h)
    logger.setLevel(logging.DEBUG if verbose else logging.INFO)
    return logger
