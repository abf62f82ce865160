"""Sharding rule and process-group helpers shared by the data-parallel wrappers.

Parity: fairscale/internal/parallel.py:21-134.  The sharding rule
(`chunk_and_pad`) defines every checkpoint layout of the library: shard ``r`` of a
tensor is elements ``[r*S, (r+1)*S)`` of its flattening with ``S = ceil(numel/world)``
and zero fill past the end.  The fused NVLink collectives use the same layout.
"""

from __future__ import annotations

import sys
from enum import Enum
from typing import TYPE_CHECKING, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

if TYPE_CHECKING:
    from torch.distributed import ProcessGroup


def shard_numel(numel: int, world_size: int) -> int:
    """Per-rank element count of the padded shard layout (``ceil(numel / world)``)."""
    return (numel + world_size - 1) // world_size if numel > 0 else 0


def chunk_and_pad(tensor: torch.Tensor, num_chunks: int) -> List[torch.Tensor]:
    """Split the flattened ``tensor`` into ``num_chunks`` equal chunks, zero-padding the tail.

    Leading chunks are views of ``tensor``; a partially filled or missing chunk is a
    fresh zero-padded tensor of the same size as chunk 0.
    """
    flat = torch.flatten(tensor)
    size = shard_numel(flat.numel(), num_chunks)
    out: List[torch.Tensor] = []
    for r in range(num_chunks):
        lo = min(r * size, flat.numel())
        hi = min(lo + size, flat.numel())
        piece = flat[lo:hi]
        if piece.numel() < size:
            padded = flat.new_zeros(size)
            if piece.numel():
                padded[: piece.numel()].copy_(piece)
            piece = padded
        out.append(piece)
    return out


def validate_process_group(device: torch.device, process_group: "ProcessGroup") -> None:
    """One-element all-gather that catches a missing ``torch.cuda.set_device`` call.

    Objects without an ``allgather`` method (dummy groups used by unit tests) are
    accepted without a check.
    """
    if not hasattr(process_group, "allgather"):
        return
    world = process_group.size()
    if "cuda" in str(device):
        probe = torch.ones(1, device=device)
        outs = list(torch.zeros(world, device=device).chunk(world))
        dist.all_gather(outs, probe, group=process_group)
        total = torch.cat(outs).sum()
        assert total == float(world), (
            f"found {total} devices in process group but world_size={world}. "
            "Check torch.cuda.set_device is called properly"
        )


def enable_pytorch_sync_bn(module: torch.nn.Module) -> None:
    """Let torch SyncBatchNorm layers run outside DDP (old torch needed a DDP hint)."""
    for layer in module.modules():
        if isinstance(layer, torch.nn.modules.SyncBatchNorm) and hasattr(layer, "_specify_ddp_gpu_num"):
            layer._specify_ddp_gpu_num(1)  # type: ignore[attr-defined]


class ProcessGroupName(str, Enum):
    default = "default"
    reduce_scatter = "reduce_scatter"


_GROUP_CACHE: Dict[Tuple[Optional[ProcessGroupName], Optional[Tuple[int, ...]]], "ProcessGroup"] = {}


def reset_process_group_cache() -> None:
    """Forget cached groups (call after ``dist.destroy_process_group``)."""
    _GROUP_CACHE.clear()


def get_process_group_cached(
    name: ProcessGroupName = ProcessGroupName.default, ranks: Optional[Sequence[int]] = None
) -> Optional["ProcessGroup"]:
    """Singleton cache of ``dist.new_group`` results keyed by ``(name, sorted ranks)``.

    Must be called collectively by all ranks the first time a key is requested.
    Inner and outer FSDP instances share the default group so they share one
    reduce-scatter bucket; the ``reduce_scatter`` name yields a second communicator so
    gradient reduction overlaps the parameter all-gathers.
    """
    if not dist.is_initialized():
        if name == ProcessGroupName.reduce_scatter and "pytest" in sys.modules:
            return None  # dummy-group unit tests
        raise RuntimeError("torch.distributed is not yet initialized but process group is requested.")

    # a destroyed-and-recreated default group invalidates everything cached before it
    world_marker = (None, None)
    if world_marker in _GROUP_CACHE and _GROUP_CACHE.get(("__world__", None)) is not dist.group.WORLD:  # type: ignore[comparison-overlap]
        _GROUP_CACHE.clear()
    if world_marker not in _GROUP_CACHE:
        default_pg = dist.new_group(ranks=ranks)
        _GROUP_CACHE[("__world__", None)] = dist.group.WORLD  # type: ignore[index,assignment]
        _GROUP_CACHE[world_marker] = default_pg
        _GROUP_CACHE[(ProcessGroupName.default, None)] = default_pg
        _GROUP_CACHE[(ProcessGroupName.default, tuple(range(dist.get_world_size())))] = default_pg

    key_ranks = None if ranks is None else tuple(sorted(set(ranks)))
    key = (name, key_ranks)
    if key not in _GROUP_CACHE:
        _GROUP_CACHE[key] = dist.new_group(ranks=key_ranks)
    return _GROUP_CACHE[key]
