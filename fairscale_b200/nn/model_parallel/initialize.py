"""Process-group grid for tensor (model), pipeline, context and data parallelism.

Parity: fairscale/nn/model_parallel/initialize.py:43-275.  Ranks are laid out as a 4-D grid
``[data, pipeline, context, model]`` with the model dimension fastest, so the ranks of one
tensor-parallel group are adjacent (on an 8xB200 box: NVSwitch neighbours whichever way the grid is cut).
The grid is held in one state object instead of module-level globals per axis.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from datetime import timedelta
from itertools import product
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from .utils import ensure_divisibility

__all__ = [
    "initialize_model_parallel",
    "model_parallel_is_initialized",
    "destroy_model_parallel",
    "get_model_parallel_group",
    "get_model_parallel_rank",
    "get_model_parallel_src_rank",
    "get_model_parallel_world_size",
    "get_data_parallel_group",
    "get_data_parallel_rank",
    "get_data_parallel_ranks",
    "get_data_parallel_world_size",
    "get_pipeline_parallel_group",
    "get_pipeline_parallel_ranks",
    "get_context_parallel_group",
    "get_context_parallel_rank",
    "get_context_parallel_ranks",
    "get_context_parallel_world_size",
]


_AXES = ("data", "pipeline", "context", "model")


@dataclass
class _Grid:
    groups: Dict[str, Any] = field(default_factory=dict)
    ranks: Dict[str, List[int]] = field(default_factory=dict)

    def clear(self) -> None:
        self.groups.clear()
        self.ranks.clear()


_STATE = _Grid()


def initialize_model_parallel(
    model_parallel_size_: int,
    pipeline_length: int = 1,
    context_parallel_size: int = 1,
    *,
    model_parallel_backend: Optional[str] = None,
    pipeline_backend: Optional[str] = None,
    cp_backend: Optional[str] = None,
    ddp_backend: Optional[str] = None,
    timeout: Optional[timedelta] = None,
) -> None:
    """Create the data / model / pipeline / context parallel groups (collective: every rank creates every group).

    With 8 ranks and ``model_parallel_size_=2``: model groups ``[0,1],[2,3],[4,5],[6,7]`` and data groups
    ``[0,2,4,6],[1,3,5,7]``.  Groups are created in the order data, model, pipeline, context.
    """
    assert dist.is_initialized()
    world = dist.get_world_size()
    mp = int(min(model_parallel_size_, world))
    ensure_divisibility(world, mp)
    ensure_divisibility(world, context_parallel_size)
    ensure_divisibility(world, mp * pipeline_length * context_parallel_size)
    rank = dist.get_rank()
    dp = world // (mp * pipeline_length * context_parallel_size)
    if rank == 0:
        print(f"> initializing model parallel with size {mp}")
        print(f"> initializing context parallel with size {context_parallel_size}")
        print(f"> initializing pipeline with size {pipeline_length}")
        print(f"> initializing ddp with size {dp}")

    assert "data" not in _STATE.groups, "data parallel group is already initialized"
    assert "model" not in _STATE.groups, "Model parallel group is already initialized"
    assert "pipeline" not in _STATE.groups, "Pipeline parallel group is already initialized"
    assert "context" not in _STATE.groups, "Context parallelism is already initialized."

    shape = (dp, pipeline_length, context_parallel_size, mp)
    grid = torch.arange(world).reshape(shape)
    mine = [int(x[0]) for x in torch.where(grid == rank)]
    backends = {"data": ddp_backend, "model": model_parallel_backend, "pipeline": pipeline_backend, "context": cp_backend}

    for axis_name in ("data", "model", "pipeline", "context"):
        axis = _AXES.index(axis_name)
        others = [a for a in range(4) if a != axis]
        for fixed in product(*(range(shape[a]) for a in others)):
            index: List[Any] = [slice(None)] * 4
            for a, v in zip(others, fixed):
                index[a] = v
            ranks = grid[tuple(index)].tolist()
            kwargs: Dict[str, Any] = {"backend": backends[axis_name]}
            if timeout is not None:
                kwargs["timeout"] = timeout
            group = dist.new_group(ranks, **kwargs)
            if all(mine[a] == v for a, v in zip(others, fixed)):
                _STATE.groups[axis_name] = group
                _STATE.ranks[axis_name] = ranks


def model_parallel_is_initialized() -> bool:
    return all(k in _STATE.groups for k in _AXES)


def _group(axis: str, msg: str) -> Any:
    assert axis in _STATE.groups, msg
    return _STATE.groups[axis]


def get_context_parallel_group() -> Any:
    return _group("context", "context parallel group is not initialized")


def get_context_parallel_ranks() -> List[int]:
    assert "context" in _STATE.ranks, "context parallel group is not initialized"
    return _STATE.ranks["context"]


def get_context_parallel_world_size() -> int:
    return dist.get_world_size(group=get_context_parallel_group())


def get_context_parallel_rank() -> int:
    return dist.get_rank(group=get_context_parallel_group())


def get_model_parallel_group() -> Any:
    return _group("model", "model parallel group is not initialized")


def get_data_parallel_group() -> Any:
    return _group("data", "data parallel group is not initialized")


def get_pipeline_parallel_group() -> Any:
    return _group("pipeline", "pipeline parallel group is not initialized")


def get_pipeline_parallel_ranks() -> List[int]:
    assert "pipeline" in _STATE.ranks, "pipeline parallel group is not initialized"
    return _STATE.ranks["pipeline"]


def get_model_parallel_world_size() -> int:
    return dist.get_world_size(group=get_model_parallel_group())


def get_model_parallel_rank() -> int:
    return dist.get_rank(group=get_model_parallel_group())


def get_model_parallel_src_rank() -> int:
    """Global rank of the first member of the caller's model-parallel group."""
    size = get_model_parallel_world_size()
    return (dist.get_rank() // size) * size


def get_data_parallel_world_size() -> int:
    return dist.get_world_size(group=get_data_parallel_group())


def get_data_parallel_rank() -> int:
    return dist.get_rank(group=get_data_parallel_group())


def get_data_parallel_ranks() -> List[int]:
    assert "data" in _STATE.ranks, "data parallel group is not initialized"
    return _STATE.ranks["data"]


def destroy_model_parallel() -> None:
    """Forget all groups (they are not destroyed; ``destroy_process_group`` does that)."""
    _STATE.clear()
