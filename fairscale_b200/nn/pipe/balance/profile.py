"""Measurements behind the automatic balancers: how long, and how much memory, each layer of a sequential model takes.

Both measurements walk the model once per pass, layer by layer, on copies of the layers (the caller's module keeps its
device, mode and gradients), feeding each layer the detached output of the previous one; ``_walk`` is that loop and the two
profilers are observers of it.  Interface of fairscale/nn/pipe/balance/profile.py:38-139.
"""

from __future__ import annotations

import copy
import time
from typing import Callable, Generator, Iterator, List, Tuple, Union

import torch
from torch import Tensor, nn

from ..microbatch import Batch

__all__: List[str] = []

Device = Union[torch.device, int, str]
Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]


def layerwise_sandbox(module: nn.Sequential, device: torch.device) -> Generator[nn.Module, None, None]:
    """One layer at a time: a deep copy, moved to ``device`` and put in training mode.  Only one copy is alive at a time."""
    for original in module:
        yield copy.deepcopy(original).to(device).train()


def detach(batch: Batch) -> None:
    """Cut the batch loose from whatever produced it, keeping each tensor's ``requires_grad``."""
    for position in range(len(batch)):
        tensor = batch[position]
        batch[position] = tensor.detach().requires_grad_(tensor.requires_grad)


def _on_device(sample: TensorOrTensors, device: torch.device, rows: slice = slice(None)) -> Batch:
    batch = Batch(sample, 0)
    for position in range(len(batch)):
        tensor = batch[position]
        batch[position] = tensor[rows].detach().to(device).requires_grad_(tensor.requires_grad)
    return batch


def _walk(module: nn.Sequential, batch: Batch, device: torch.device, run_layer: Callable[[int, nn.Module, Batch], Batch]) -> Iterator[int]:
    """Feed ``batch`` through sandboxed copies of the layers; ``run_layer(index, layer, detached input)`` returns the output."""
    for index, layer in enumerate(layerwise_sandbox(module, device)):
        detach(batch)
        batch = run_layer(index, layer, batch)
        yield index


def profile_times(module: nn.Sequential, sample: TensorOrTensors, timeout: float, device: torch.device) -> List[int]:
    """Microseconds of forward + backward per layer, summed over as many passes as fit into ``timeout`` seconds."""
    if any(p.grad is not None for p in module.parameters()):
        raise ValueError("some parameter already has gradient")
    wait = (lambda: torch.cuda.synchronize(device)) if device.type == "cuda" else (lambda: None)
    seconds = [0.0] * len(module)

    def timed(index: int, layer: nn.Module, batch: Batch) -> Batch:
        wait()
        started = time.time()
        out = batch.call(layer)
        roots = tuple(y for y in out if y.requires_grad)
        if roots:
            torch.autograd.backward(roots, roots)  # any gradient of the right shape will do for timing
        wait()
        seconds[index] += time.time() - started
        return out

    deadline = time.time() + timeout
    first_pass = True
    while first_pass or time.time() < deadline:
        first_pass = False
        for _ in _walk(module, _on_device(sample, device), device, timed):
            pass
    return [int(s * 1_000_000) for s in seconds]


def profile_sizes(module: nn.Sequential, input: TensorOrTensors, chunks: int, param_scale: float, device: torch.device) -> List[int]:
    """Bytes per layer: what one micro-batch keeps alive for backward plus ``param_scale`` times the parameter bytes
    (parameters, gradients and optimizer state in one factor).  Needs an allocator that reports its usage: CUDA only."""
    if device.type != "cuda":
        raise ValueError("size profiler supports only CUDA device")
    rows_per_microbatch = Batch(input, 0)[0].size(0) / chunks  # measured on one row, scaled to a micro-batch
    sizes: List[int] = []

    def weighed(index: int, layer: nn.Module, batch: Batch) -> Batch:
        held_before = torch.cuda.memory_allocated(device)
        out = batch.call(layer)
        kept = torch.cuda.memory_allocated(device) - held_before
        parameter_bytes = sum(p.untyped_storage().size() for p in layer.parameters())
        sizes.append(int(kept * rows_per_microbatch + parameter_bytes * param_scale))
        return out

    for _ in _walk(module, _on_device(input, device, rows=slice(0, 1)), device, weighed):
        pass
    return sizes
