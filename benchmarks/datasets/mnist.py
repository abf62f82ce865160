"""MNIST-shaped data for the OSS benchmark.  Offline: synthetic 1x28x28 images whose label is a fixed linear function
of the pixels, so a model can actually fit it and the loss regression check stays meaningful."""

import torch
from torch.utils.data import TensorDataset


def setup_cached_mnist(n: int = 8192, seed: int = 0) -> TensorDataset:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, 1, 28, 28, generator=g)
    w = torch.randn(28 * 28, 10, generator=g)
    y = (x.view(n, -1) @ w).argmax(-1)
    return TensorDataset(x, y)
