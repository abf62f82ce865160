"""How much of a tensor's energy sits in its largest entries (parity: .../wgit/signal_sparsity_profiling.py:12-62)."""

from typing import List

import torch
from torch import Tensor


class EnergyConcentrationProfile:
    """For every percentage p in ``top_k_percents``: the share of total |x| held by the top p % of entries along ``dim``."""

    def __init__(self, dim: int, top_k_percents: List[float]) -> None:
        self.dim = dim
        for p in top_k_percents:
            assert 0.0 < p <= 100.0, p
        self.percents = top_k_percents

    def measure(self, in_tensor: Tensor) -> List[Tensor]:
        assert in_tensor.is_floating_point(), in_tensor.dtype
        abs_t = in_tensor.abs()
        sorted_t = abs_t.sort(dim=self.dim, descending=True).values
        total = sorted_t.sum()
        n = in_tensor.shape[self.dim]
        out = []
        for p in self.percents:
            k = max(1, round(n * p / 100.0))
            out.append(sorted_t.narrow(self.dim, 0, k).sum() / total)
        return out

    def measure_fft(self, in_tensor: Tensor) -> List[Tensor]:
        """Same, on the magnitude of the real part of the tensor's FFT along ``dim``."""
        return self.measure(torch.fft.fft(in_tensor, dim=self.dim).real)
