"""Flat buffers backing ``param.data`` (ParamBucket) or ``param.grad`` (GradBucket).

API parity: fairscale/nn/misc/param_bucket.py:11-248.  Used by OSS (one parameter
bucket per owner rank, broadcast after the step) and ShardedDataParallel (one gradient
bucket per owner rank, reduced once all its gradients have checked in).

Entries can be aligned (``align`` elements) so that every tensor starts on a 16-byte
boundary: the multi-tensor Adam kernel then uses 128-bit loads on each member and a
whole bucket is a legal source for bulk copies.
"""

from __future__ import annotations

from typing import Any, Callable, Iterable, List, Optional, Union

import torch


def _round_up(n: int, align: int) -> int:
    return (n + align - 1) // align * align if align > 1 else n


class Bucket:
    """A flat tensor and the list of tensors whose storage it provides."""

    def __init__(self, size: int, dtype: torch.dtype, device: torch.device, align: int = 1) -> None:
        self._params: List[torch.Tensor] = []
        self._param_ids: List[int] = []
        self._fill = 0
        self._align = max(1, int(align))
        self.buffer: torch.Tensor = torch.zeros(size, dtype=dtype, device=device)

    @staticmethod
    def required_size(tensors: Iterable[torch.Tensor], align: int = 1) -> int:
        """Buffer size needed to hold ``tensors`` with each entry aligned to ``align`` elements."""
        return sum(_round_up(t.numel(), align) for t in tensors)

    def _claim(self, numel: int) -> slice:
        lo = self._fill
        hi = lo + numel
        assert hi <= self.buffer.numel(), "bucket overflow"
        self._fill = _round_up(hi, self._align)
        return slice(lo, hi)

    def to(  # type: ignore[no-untyped-def]
        self,
        device: Optional[Union[int, torch.device]],
        dtype: Optional[torch.dtype] = None,
        non_blocking: bool = False,
        keep_param_alignment: bool = True,
    ):
        assert self.buffer is not None, "Cannot move a collapsed bucket, please rebuild it"
        self.buffer = self.buffer.to(device, dtype, non_blocking)


class ParamBucket(Bucket):
    """Parameters whose ``.data`` are views of one flat buffer."""

    def to(  # type: ignore[no-untyped-def,override]
        self,
        device: Optional[Union[int, torch.device]],
        dtype: Optional[torch.dtype] = None,
        non_blocking: bool = False,
        keep_param_alignment: bool = True,
    ):
        super().to(device, dtype, non_blocking)
        if keep_param_alignment:
            self._reattach_params()

    @torch.no_grad()
    def add_param(self, param: torch.Tensor) -> None:
        """Copy ``param`` into the buffer and make ``param.data`` a view of it."""
        assert id(param) not in self._param_ids, "The same param cannot be checked in twice"
        self._add_param_as_view(param)
        self._params.append(param)
        self._param_ids.append(id(param))

    @torch.no_grad()
    def _add_param_as_view(self, param: torch.Tensor, keep_existing_value: bool = True) -> None:
        assert self.buffer is not None
        assert param.dtype == self.buffer.dtype, (
            f"Different types for the bucket and the param, cannot proceed: {param.dtype} - {self.buffer.dtype}"
        )
        assert param.device == self.buffer.device, (
            f"Different devices for the bucket and the param, cannot proceed: {param.device} - {self.buffer.device}"
        )
        window = self.buffer[self._claim(param.numel())]
        if keep_existing_value:
            window.copy_(param.data.flatten())
        param.data = window.view_as(param.data)

    @torch.no_grad()
    def _reattach_params(self) -> None:
        assert len(self._params) > 0
        self._fill = 0
        for p in self._params:
            if p.dtype != self.buffer.dtype:
                p.data = p.data.to(self.buffer.dtype)
            self._add_param_as_view(p, keep_existing_value=False)


class GradBucket(Bucket):
    """Gradients whose storage is one flat buffer that is reduced to ``destination`` as a whole."""

    def __init__(self, size: int, dtype: torch.dtype, device: torch.device, destination: int, align: int = 1) -> None:
        super().__init__(size, dtype, device, align)
        self._max_size = size
        self._is_collapsed = False
        self.params_checked_in = 0
        self.destination = destination
        self.sent = True
        self.callback: Optional[Callable[[Any], None]] = None

    def reset_checked_in(self) -> None:
        self.params_checked_in = 0
        self.sent = False

    @property
    def all_checked_in(self) -> bool:
        return len(self._params) == self.params_checked_in

    def can_add_grad_view(self, param: torch.Tensor) -> bool:
        return self._fill + param.numel() < self._max_size and id(param) not in self._param_ids

    def to(  # type: ignore[no-untyped-def,override]
        self,
        device: Optional[Union[int, torch.device]],
        dtype: Optional[torch.dtype] = None,
        non_blocking: bool = False,
        keep_param_alignment: bool = True,
    ):
        if self._is_collapsed:
            self.rebuild()
        super().to(device, dtype, non_blocking)
        if keep_param_alignment:
            self._reattach_grads()

    def zero(self) -> None:
        self.buffer.fill_(0.0)

    @torch.no_grad()
    def add_grad(self, param: torch.Tensor) -> None:
        """Make ``param.grad`` a view of the buffer (allocating a zero grad if there is none)."""
        assert id(param) not in self._param_ids, "The same gradients cannot be checked in twice"
        if param.grad is None:
            param.grad = torch.zeros_like(param)
        self._add_grad_as_view(param)
        self._params.append(param)
        self._param_ids.append(id(param))

    @torch.no_grad()
    def collapse(self) -> None:
        """Free the buffer; gradients of the members become ``None`` until :meth:`rebuild`."""
        if self._is_collapsed:
            return
        for p in self._params:
            assert p.grad is not None
            p.grad.detach_()
            p.grad = None
        self.buffer = torch.zeros(0, dtype=self.buffer.dtype, device=self.buffer.device)
        self._fill = 0
        self.params_checked_in = 0
        self._is_collapsed = True

    @torch.no_grad()
    def rebuild(self) -> None:
        assert len(self._params) > 0
        if not self._is_collapsed:
            return
        self.buffer = torch.zeros(self._max_size, dtype=self._params[0].dtype, device=self._params[0].device)
        self._fill = 0
        for p in self._params:
            self._add_grad_as_view(p)
        self._is_collapsed = False

    @torch.no_grad()
    def shrink(self) -> None:
        """Trim the buffer to the part in use."""
        assert self.buffer.numel() > 0, "Cannot shrink a collapsed bucket, please rebuild"
        self.buffer = self.buffer[: self._fill].clone()
        self._fill = 0
        for p in self._params:
            self._add_grad_as_view(p)
        self._max_size = self._fill

    @torch.no_grad()
    def _reattach_grads(self) -> None:
        assert len(self._params) > 0
        self._fill = 0
        for p in self._params:
            self._add_grad_as_view(p, keep_existing_value=False)

    @torch.no_grad()
    def _add_grad_as_view(self, param: torch.Tensor, keep_existing_value: bool = True) -> None:
        assert self.buffer.numel() > 0, "Cannot add a gradient to a collapsed bucket, please rebuild"
        assert param.dtype == self.buffer.dtype
        assert param.device == self.buffer.device
        window = self.buffer[self._claim(param.numel())]
        if param.grad is not None:
            if keep_existing_value:
                window.copy_(param.grad.data.flatten())
            param.grad.data = window.view_as(param.data)
        else:
            param.grad = window.view_as(param.data)
