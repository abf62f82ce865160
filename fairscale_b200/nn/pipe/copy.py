"""Autograd-aware movement of micro-batches between the devices of a pipeline.

``Copy`` transfers tensors from the device of ``prev_stream`` to the device of ``next_stream``; the copy is issued
while both copy streams are current, so neither compute stream is involved.  ``Wait`` only synchronises: the stream that
is going to use the tensors waits for the stream that produced them.  In backward each does the mirror image (gradients
travel from ``next`` to ``prev``; the wait is reversed).  Same roles as fairscale/nn/pipe/copy.py:32-108.
"""

from __future__ import annotations

from typing import Any, List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from .stream import AbstractStream, current_stream, get_device, record_stream, use_stream, wait_stream

__all__: List[str] = []

Tensors = Tuple[Tensor, ...]


class Context:
    """Typing aid: the stream pair an autograd context of this module carries."""

    prev_stream: AbstractStream
    next_stream: AbstractStream


def _transfer(tensors: Sequence[Tensor], src: AbstractStream, dst: AbstractStream) -> List[Tensor]:
    """``tensors`` (resident on ``src``'s device, produced / consumed on that device's compute stream) copied to
    ``dst``'s device.  The caching allocator is told which foreign streams touch which block."""
    src_compute = current_stream(get_device(src))
    dst_device = get_device(dst)
    moved: List[Tensor] = []
    with use_stream(src), use_stream(dst):
        for t in tensors:
            m = t.to(dst_device, non_blocking=True)
            record_stream(t, src)          # born on the compute stream, read by the copy stream
            record_stream(m, src_compute)  # kept alive as long as the side that owns the graph may refer to it
            moved.append(m)
    return moved


class Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, prev_stream: AbstractStream, next_stream: AbstractStream, *input: Tensor) -> Tensors:  # type: ignore[override]
        ctx.streams = (prev_stream, next_stream)
        return tuple(_transfer(input, prev_stream, next_stream))

    @staticmethod
    def backward(ctx: Any, *grad_output: Tensor) -> Tuple[Optional[Tensor], ...]:  # type: ignore[override]
        prev_stream, next_stream = ctx.streams
        return (None, None, *_transfer(grad_output, next_stream, prev_stream))


class Wait(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, prev_stream: AbstractStream, next_stream: AbstractStream, *input: Tensor) -> Tensors:  # type: ignore[override]
        ctx.streams = (prev_stream, next_stream)
        wait_stream(next_stream, prev_stream)
        return tuple(t.detach() for t in input)

    @staticmethod
    def backward(ctx: Any, *grad_input: Tensor) -> Tuple[Optional[Tensor], ...]:  # type: ignore[override]
        prev_stream, next_stream = ctx.streams
        wait_stream(prev_stream, next_stream)
        return (None, None, *grad_input)
