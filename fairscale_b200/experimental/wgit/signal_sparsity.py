"""Frequency-domain top-k sparsification of tensors: signal sparse tensor (SST) + delta sparse tensor (DST).

Capability parity with fairscale/experimental/wgit/signal_sparsity.py:14-446.  ``dense -> transform -> top-k`` gives
the SST, ``dense - inverse(SST) -> top-k`` gives the DST, and ``inverse(SST) + DST`` is the lossy reconstruction.
Both the FFT and the DCT (type II, computed through an FFT of the mirrored signal; the reference leaves DCT
unimplemented) are available.
"""

from __future__ import annotations

from enum import Enum
import math
from typing import Optional, Tuple

import torch
from torch import Tensor


def _get_k_for_topk(topk_percent: Optional[float], top_k_element: Optional[int], top_k_total_size: int) -> int:
    if top_k_element is None:
        assert topk_percent is not None
        return max(1, int(top_k_total_size * topk_percent / 100.0))
    return min(top_k_element, top_k_total_size)


def _scatter_topk_to_sparse_tensor(top_k_tensor: Tensor, to_be_sparsify_tensor: Tensor, k: int, dim: Optional[int]) -> Tensor:
    """Keep the entries of ``to_be_sparsify_tensor`` at the positions of the ``k`` largest entries of
    ``top_k_tensor`` along ``dim`` (over the flattened tensor when ``dim`` is None); zero elsewhere."""
    assert top_k_tensor.shape == to_be_sparsify_tensor.shape, "shape mismatch"
    shape = top_k_tensor.shape
    if dim is None:
        top_k_tensor, to_be_sparsify_tensor, d = top_k_tensor.reshape(-1), to_be_sparsify_tensor.reshape(-1), 0
    else:
        d = dim
    idx = torch.topk(top_k_tensor, k, dim=d, sorted=False).indices
    out = torch.zeros_like(to_be_sparsify_tensor)
    out.scatter_(d, idx, to_be_sparsify_tensor.gather(d, idx))
    return out.reshape(shape)


def _top_k_total_size(tensor: Tensor, topk_dim: Optional[int]) -> int:
    return tensor.shape[topk_dim] if topk_dim is not None else tensor.numel()


def _is_sparsity_zero(dense: Tensor, topk_percent: Optional[float], topk_element: Optional[int], top_k_dim: Optional[int]) -> bool:
    if topk_percent is None and topk_element is None:
        return False
    total = _top_k_total_size(dense, top_k_dim)
    return _get_k_for_topk(topk_percent, topk_element, total) == total


def _fft_transform(dense: Tensor, dim: Optional[int]) -> Tensor:
    return torch.fft.fft(dense, dim=dim) if dim is not None else torch.fft.fft(dense.reshape(-1)).reshape(dense.shape)


def _ifft_transform(sst: Tensor, dim: Optional[int]) -> Tensor:
    return torch.fft.ifft(sst, dim=dim) if dim is not None else torch.fft.ifft(sst.reshape(-1)).reshape(sst.shape)


def _dct_last(x: Tensor) -> Tensor:
    """Orthonormal DCT-II along the last dimension via one FFT of length N (Makhoul's reordering)."""
    n = x.shape[-1]
    v = torch.cat([x[..., ::2], x[..., 1::2].flip(-1)], dim=-1)
    V = torch.fft.fft(v.to(torch.float64 if x.dtype == torch.float64 else torch.float32), dim=-1)
    k = torch.arange(n, device=x.device, dtype=V.real.dtype)
    W = torch.exp(-1j * math.pi * k / (2 * n))
    out = (V * W).real * 2
    out[..., 0] /= math.sqrt(n) * 2
    out[..., 1:] /= math.sqrt(n / 2) * 2
    return out.to(x.dtype)


def _idct_last(X: Tensor) -> Tensor:
    n = X.shape[-1]
    f = X.to(torch.float64 if X.dtype == torch.float64 else torch.float32).clone()
    f[..., 0] *= math.sqrt(n) * 2
    f[..., 1:] *= math.sqrt(n / 2) * 2
    k = torch.arange(n, device=X.device, dtype=f.dtype)
    W = torch.exp(1j * math.pi * k / (2 * n))
    flipped = torch.cat([torch.zeros_like(f[..., :1]), -f.flip(-1)[..., :-1]], dim=-1)
    V = (f + 1j * flipped) * W / 2
    v = torch.fft.ifft(V, dim=-1).real
    x = torch.empty_like(v)
    x[..., ::2] = v[..., : (n + 1) // 2]
    x[..., 1::2] = v[..., (n + 1) // 2 :].flip(-1)
    return x.to(X.dtype)


def _dct_transform(dense: Tensor, dim: Optional[int]) -> Tensor:
    if dim is None:
        return _dct_last(dense.reshape(-1)).reshape(dense.shape)
    return _dct_last(dense.transpose(dim, -1)).transpose(dim, -1)


def _idct_transform(sst: Tensor, dim: Optional[int]) -> Tensor:
    sst = sst.real if sst.is_complex() else sst
    if dim is None:
        return _idct_last(sst.reshape(-1)).reshape(sst.shape)
    return _idct_last(sst.transpose(dim, -1)).transpose(dim, -1)


class Algo(Enum):
    FFT = 0
    DCT = 1


class SignalSparsity:
    """One sparsification configuration.  Exactly one of ``*_top_k_element`` / ``*_top_k_percent`` may be set for
    the SST and for the DST; a ``*_top_k_dim`` of None means top-k over the flattened tensor."""

    def __init__(self, algo: Algo = Algo.FFT, sst_top_k_dim: Optional[int] = -1, sst_top_k_element: Optional[int] = None,
                 sst_top_k_percent: Optional[float] = None, dst_top_k_dim: Optional[int] = -1,
                 dst_top_k_element: Optional[int] = None, dst_top_k_percent: Optional[float] = None) -> None:
        self._sst_top_k_dim, self._sst_top_k_element, self._sst_top_k_percent = sst_top_k_dim, sst_top_k_element, sst_top_k_percent
        self._dst_top_k_dim, self._dst_top_k_element, self._dst_top_k_percent = dst_top_k_dim, dst_top_k_element, dst_top_k_percent
        self._validate_conf()
        self._transform, self._inverse_transform = (_fft_transform, _ifft_transform) if algo is Algo.FFT else (_dct_transform, _idct_transform)

    @property
    def _sst_enabled(self) -> bool:
        return self._sst_top_k_element is not None or self._sst_top_k_percent is not None

    @property
    def _dst_enabled(self) -> bool:
        return self._dst_top_k_element is not None or self._dst_top_k_percent is not None

    def _validate_conf(self) -> None:
        for what, el, pc in (("sst", self._sst_top_k_element, self._sst_top_k_percent), ("dst", self._dst_top_k_element, self._dst_top_k_percent)):
            if el is not None and pc is not None:
                raise ValueError(f"top_k_element and top_k_percent can't be both set ({what}: element={el}, percent={pc})")
            if pc is not None and not (0.0 < pc <= 100.0):
                raise ValueError(f"top_k_percent for {what} has to be in the interval (0, 100], got {pc}")
            if el is not None and el <= 0:
                raise ValueError(f"top_k_element for {what} has to be greater than 0, got {el}")

    def dense_to_sst(self, dense: Tensor) -> Optional[Tensor]:
        """Transform and keep the top-k coefficients (by magnitude of the real part); same shape, frequency domain."""
        if not self._sst_enabled:
            return None
        k = _get_k_for_topk(self._sst_top_k_percent, self._sst_top_k_element, _top_k_total_size(dense, self._sst_top_k_dim))
        freq = self._transform(dense, dim=self._sst_top_k_dim)
        return _scatter_topk_to_sparse_tensor(freq.real.abs(), freq, k, dim=self._sst_top_k_dim)

    def dense_sst_to_dst(self, dense: Tensor, sst: Optional[Tensor]) -> Optional[Tensor]:
        """Top-k (by magnitude) of what the SST fails to reconstruct."""
        if not self._dst_enabled:
            return None
        if sst is None:
            sst = torch.zeros_like(dense, dtype=torch.complex64)
        if dense.shape != sst.shape:
            raise ValueError("dense and sst have different shapes!")
        k = _get_k_for_topk(self._dst_top_k_percent, self._dst_top_k_element, _top_k_total_size(dense, self._dst_top_k_dim))
        delta = dense - self.sst_dst_to_dense(sst)
        return _scatter_topk_to_sparse_tensor(delta.abs(), delta, k, dim=self._dst_top_k_dim)

    def sst_dst_to_dense(self, sst: Optional[Tensor], dst: Optional[Tensor] = None) -> Tensor:
        assert not (sst is None and dst is None), "both-None-case is not useful"
        if sst is None:
            return dst  # type: ignore[return-value]
        rt = torch.real(self._inverse_transform(sst, dim=self._sst_top_k_dim)) if sst.is_complex() else self._inverse_transform(sst, dim=self._sst_top_k_dim)
        return rt + dst if dst is not None else rt

    def lossy_compress(self, dense: Tensor) -> Tuple[Tensor, Optional[Tensor], Optional[Tensor]]:
        """(reconstruction, sst, dst); the input itself when nothing would be dropped."""
        if _is_sparsity_zero(dense, self._sst_top_k_percent, self._sst_top_k_element, self._sst_top_k_dim) and _is_sparsity_zero(
            dense, self._dst_top_k_percent, self._dst_top_k_element, self._dst_top_k_dim
        ):
            return dense, None, dense
        sst = self.dense_to_sst(dense)
        dst = self.dense_sst_to_dst(dense, sst)
        return self.sst_dst_to_dense(sst, dst), sst, dst


def random_sparse_mask(dense: Tensor, percent: float, dim: int) -> Tensor:
    """0/1 mask with ``percent`` % ones at random positions along ``dim``."""
    assert 0 < percent <= 100, percent
    k = _get_k_for_topk(percent, None, dense.shape[dim])
    return _scatter_topk_to_sparse_tensor(torch.rand_like(dense), torch.ones_like(dense), k, dim)
