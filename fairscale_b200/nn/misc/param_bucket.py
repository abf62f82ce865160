"""Flat buffers that own the storage of many small tensors.

A :class:`ParamBucket` backs ``param.data`` of its members, a :class:`GradBucket` backs ``param.grad``.  OSS keeps one
parameter bucket per (device, owner rank) and publishes the owner's updated values with one collective on the flat
buffer; ShardedDataParallel keeps one gradient bucket per (device, owner rank) and reduces it once every member's
gradient has checked in.  Public interface of fairscale/nn/misc/param_bucket.py:11-248.

Layout: the bucket keeps an offset table (one ``_Slot`` per member).  Offsets are multiples of ``align`` elements, so
with ``align`` covering 16 bytes every member can be read with 128-bit loads by the multi-tensor kernels and the whole
buffer is a legal operand of the NVLink collectives.  ``allocator(numel, dtype, device)`` lets the caller place the
buffer somewhere special - the symmetric heap of an NVLink workspace, so that peers can pull the bucket directly.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Union

import torch

Allocator = Callable[[int, torch.dtype, torch.device], torch.Tensor]


def _aligned(n: int, align: int) -> int:
    return -(-n // align) * align


@dataclass
class _Slot:
    tensor: torch.Tensor  # the member parameter
    offset: int           # first element of its window in the flat buffer
    numel: int


class Bucket:
    """The flat buffer and its offset table; subclasses say which attribute of a member the windows back."""

    def __init__(self, size: int, dtype: torch.dtype, device: torch.device, align: int = 1, allocator: Optional[Allocator] = None) -> None:
        self._align = max(int(align), 1)
        self._allocator = allocator
        self._slots: List[_Slot] = []
        self._by_id: Dict[int, _Slot] = {}
        self._cursor = 0  # first free element
        self.buffer: torch.Tensor = self._allocate(size, dtype, torch.device(device))

    # -- storage
    def _allocate(self, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        if self._allocator is not None:
            return self._allocator(numel, dtype, device).zero_()
        return torch.zeros(numel, dtype=dtype, device=device)

    @staticmethod
    def required_size(tensors: Iterable[torch.Tensor], align: int = 1) -> int:
        """Elements a bucket needs to hold ``tensors`` when every window starts on a multiple of ``align``."""
        return sum(_aligned(t.numel(), max(int(align), 1)) for t in tensors)

    # -- offset table
    @property
    def _params(self) -> List[torch.Tensor]:
        return [s.tensor for s in self._slots]

    def _holds(self, tensor: torch.Tensor) -> bool:
        return id(tensor) in self._by_id

    def _reserve(self, tensor: torch.Tensor) -> _Slot:
        end = self._cursor + tensor.numel()
        assert end <= self.buffer.numel(), "bucket overflow"
        slot = _Slot(tensor, self._cursor, tensor.numel())
        self._cursor = _aligned(end, self._align)
        self._slots.append(slot)
        self._by_id[id(tensor)] = slot
        return slot

    def _window(self, slot: _Slot) -> torch.Tensor:
        return self.buffer[slot.offset : slot.offset + slot.numel].view(slot.tensor.shape)

    def _check_compatible(self, tensor: torch.Tensor) -> None:
        assert tensor.dtype == self.buffer.dtype, (
            f"Different types for the bucket and the param, cannot proceed: {tensor.dtype} - {self.buffer.dtype}"
        )
        assert tensor.device == self.buffer.device, (
            f"Different devices for the bucket and the param, cannot proceed: {tensor.device} - {self.buffer.device}"
        )

    # -- what a subclass backs (``data`` or ``grad``)
    def _attach(self, slot: _Slot, carry_value: bool) -> None:
        raise NotImplementedError

    def _reattach_all(self, carry_value: bool) -> None:
        for slot in self._slots:
            self._attach(slot, carry_value)

    def to(  # type: ignore[no-untyped-def]
        self,
        device: Optional[Union[int, torch.device]],
        dtype: Optional[torch.dtype] = None,
        non_blocking: bool = False,
        keep_param_alignment: bool = True,
    ):
        """Move / cast the flat buffer; with ``keep_param_alignment`` the members are re-pointed at the new buffer."""
        assert self.buffer is not None, "Cannot move a collapsed bucket, please rebuild it"
        self.buffer = self.buffer.to(device, dtype, non_blocking)
        if keep_param_alignment and self._slots:
            self._reattach_all(carry_value=False)


class ParamBucket(Bucket):
    """``param.data`` of every member is a window of the flat buffer."""

    @torch.no_grad()
    def add_param(self, param: torch.Tensor) -> None:
        """Copy ``param`` into the next free window and re-point ``param.data`` at it."""
        assert not self._holds(param), "The same param cannot be checked in twice"
        self._check_compatible(param)
        self._attach(self._reserve(param), carry_value=True)

    @torch.no_grad()
    def _attach(self, slot: _Slot, carry_value: bool) -> None:
        param = slot.tensor
        if param.dtype != self.buffer.dtype:  # the bucket was cast (OSS broadcasts in fp16): the member follows
            param.data = param.data.to(self.buffer.dtype)
        window = self._window(slot)
        if carry_value:
            window.copy_(param.data)
        param.data = window


class GradBucket(Bucket):
    """``param.grad`` of every member is a window of the flat buffer, which is reduced to rank ``destination`` as a
    whole.  The buffer can be released between steps (:meth:`collapse` / :meth:`rebuild`) and trimmed to the part in
    use (:meth:`shrink`)."""

    def __init__(self, size: int, dtype: torch.dtype, device: torch.device, destination: int, align: int = 1,
                 allocator: Optional[Allocator] = None) -> None:
        super().__init__(size, dtype, device, align, allocator)
        self._max_size = size
        self._is_collapsed = False
        self.destination = destination
        self.params_checked_in = 0  # members whose gradient is complete in the current backward
        self.sent = True            # the reduction of the current backward has been issued
        self.callback: Optional[Callable[[Any], None]] = None

    # -- per-backward bookkeeping
    def reset_checked_in(self) -> None:
        self.params_checked_in, self.sent = 0, False

    @property
    def all_checked_in(self) -> bool:
        return self.params_checked_in == len(self._slots)

    def can_add_grad_view(self, param: torch.Tensor) -> bool:
        """Room left for ``param`` and not a member yet."""
        return self._cursor + param.numel() < self._max_size and not self._holds(param)

    def zero(self) -> None:
        self.buffer.zero_()

    # -- membership
    @torch.no_grad()
    def add_grad(self, param: torch.Tensor) -> None:
        """Make ``param.grad`` a window of the buffer; an existing gradient keeps its value, a missing one starts at 0."""
        assert not self._holds(param), "The same gradients cannot be checked in twice"
        assert not self._is_collapsed, "Cannot add a gradient to a collapsed bucket, please rebuild"
        self._check_compatible(param)
        self._attach(self._reserve(param), carry_value=True)

    @torch.no_grad()
    def _attach(self, slot: _Slot, carry_value: bool) -> None:
        assert self.buffer.numel() > 0, "Cannot add a gradient to a collapsed bucket, please rebuild"
        param, window = slot.tensor, self._window(slot)
        if param.grad is None:
            param.grad = window  # the buffer is zero-initialised
            return
        if carry_value:
            window.copy_(param.grad)
        param.grad.data = window

    @torch.no_grad()
    def readopt_grad(self, param: torch.Tensor) -> None:
        """If ``param.grad`` was replaced since it joined (an optimizer's ``zero_grad(set_to_none=True)`` drops it and
        autograd then allocates a fresh one), move the new gradient into its window and point ``param.grad`` back."""
        slot = self._by_id[id(param)]
        grad = param.grad
        if grad is None or self._is_collapsed:
            return
        if grad.data_ptr() != self.buffer.data_ptr() + slot.offset * self.buffer.element_size():
            window = self._window(slot)
            window.copy_(grad)
            param.grad = window

    # -- buffer life cycle
    def to(  # type: ignore[no-untyped-def,override]
        self,
        device: Optional[Union[int, torch.device]],
        dtype: Optional[torch.dtype] = None,
        non_blocking: bool = False,
        keep_param_alignment: bool = True,
    ):
        if self._is_collapsed:
            self.rebuild()
        super().to(device, dtype, non_blocking, keep_param_alignment)

    @torch.no_grad()
    def collapse(self) -> None:
        """Release the buffer; the members' gradients become ``None`` until :meth:`rebuild`."""
        if self._is_collapsed:
            return
        for slot in self._slots:
            assert slot.tensor.grad is not None
            slot.tensor.grad = None
        self.buffer = torch.zeros(0, dtype=self.buffer.dtype, device=self.buffer.device)
        self.params_checked_in = 0
        self._is_collapsed = True

    @torch.no_grad()
    def rebuild(self) -> None:
        """Undo :meth:`collapse`: a fresh zero buffer with the same offset table."""
        assert len(self._slots) > 0
        if not self._is_collapsed:
            return
        first = self._slots[0].tensor
        self.buffer = self._allocate(self._max_size, first.dtype, first.device)
        self._is_collapsed = False
        self._reattach_all(carry_value=True)

    @torch.no_grad()
    def shrink(self) -> None:
        """Cut the buffer down to the windows handed out so far (values kept)."""
        assert self.buffer.numel() > 0, "Cannot shrink a collapsed bucket, please rebuild"
        self._max_size = self._cursor
        if self._allocator is not None:
            trimmed = self._allocator(self._cursor, self.buffer.dtype, self.buffer.device)
            trimmed.copy_(self.buffer[: self._cursor])
            self.buffer = trimmed
        else:
            self.buffer = self.buffer[: self._cursor].clone()
        self._reattach_all(carry_value=False)
