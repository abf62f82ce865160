"""Per-layer time / memory profiling used by the auto-balancers (parity: fairscale/nn/pipe/balance/profile.py:38-139)."""

from __future__ import annotations

import copy
import time
from typing import Generator, List, Tuple, Union

import torch
from torch import Tensor, nn

from ..microbatch import Batch

__all__: List[str] = []

Device = Union[torch.device, int, str]
Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]


def layerwise_sandbox(module: nn.Sequential, device: torch.device) -> Generator[nn.Module, None, None]:
    """Yield a training-mode copy of each layer on ``device``; the original module is left untouched."""
    for layer in module:
        clone = copy.deepcopy(layer)
        clone.to(device)
        clone.train()
        yield clone


def detach(batch: Batch) -> None:
    for i, x in enumerate(batch):
        batch[i] = x.detach().requires_grad_(x.requires_grad)


def _sync(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize(device)


def profile_times(module: nn.Sequential, sample: TensorOrTensors, timeout: float, device: torch.device) -> List[int]:
    """Forward+backward microseconds per layer, accumulated over repeated runs until ``timeout`` seconds passed."""
    if any(p.grad is not None for p in module.parameters()):
        raise ValueError("some parameter already has gradient")
    batch = Batch(sample, 0)
    for i, x in enumerate(batch):
        batch[i] = x.detach().to(device).requires_grad_(x.requires_grad)
    elapsed: List[List[float]] = [[] for _ in module]
    begun = time.time()
    while time.time() - begun < timeout:
        cur = batch
        for i, layer in enumerate(layerwise_sandbox(module, device)):
            detach(cur)
            _sync(device)
            t0 = time.time()
            cur = cur.call(layer)
            backward_from = tuple(y for y in cur if y.requires_grad)
            if backward_from:
                torch.autograd.backward(backward_from, backward_from)
            _sync(device)
            elapsed[i].append(time.time() - t0)
    return [int(sum(ts) * 1_000_000) for ts in elapsed]


def profile_sizes(module: nn.Sequential, input: TensorOrTensors, chunks: int, param_scale: float, device: torch.device) -> List[int]:
    """Bytes per layer: activation memory of one micro-batch + ``param_scale`` x parameter bytes (CUDA only)."""
    if device.type != "cuda":
        raise ValueError("size profiler supports only CUDA device")
    batch = Batch(input, 0)
    sizes: List[int] = []
    latent_scale = batch[0].size(0) / chunks
    for i, x in enumerate(batch):
        batch[i] = x[:1].detach().to(device).requires_grad_(x.requires_grad)
    for layer in layerwise_sandbox(module, device):
        detach(batch)
        before = torch.cuda.memory_allocated(device)
        batch = batch.call(layer)
        after = torch.cuda.memory_allocated(device)
        latent = after - before
        params = sum(p.untyped_storage().size() for p in layer.parameters())
        sizes.append(int(latent * latent_scale + params * param_scale))
    return sizes
