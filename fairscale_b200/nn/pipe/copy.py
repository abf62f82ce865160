"""Stream-aware copies between pipeline stages (parity: fairscale/nn/pipe/copy.py:43-133).

``Copy`` moves a micro-batch to the next stage's device on a dedicated copy stream (peer-to-peer over NVLink
for CUDA devices of one box); ``Wait`` makes a stream wait for another without moving data.  Both mirror
themselves in backward and keep the caching allocator informed with ``record_stream``.
"""

from __future__ import annotations

from collections import deque
from typing import Deque, List, Optional, Tuple

import torch
from torch import Tensor

from .stream import AbstractStream, current_stream, get_device, record_stream, use_stream, wait_stream

__all__: List[str] = []

Tensors = Tuple[Tensor, ...]


class Context:
    prev_stream: AbstractStream
    next_stream: AbstractStream


class Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Context, prev_stream: AbstractStream, next_stream: AbstractStream, *input: Tensor) -> Tensors:  # type: ignore[override]
        ctx.prev_stream, ctx.next_stream = prev_stream, next_stream
        out: List[Tensor] = []
        produced_on = current_stream(get_device(prev_stream))
        with use_stream(prev_stream), use_stream(next_stream):
            for x in input:
                y = x.to(get_device(next_stream), non_blocking=True)
                out.append(y)
                record_stream(x, prev_stream)  # x was allocated on the compute stream, read on prev_stream
                record_stream(y, produced_on)  # y is allocated on next_stream, consumed later on the compute stream
        return tuple(out)

    @staticmethod
    def backward(ctx: Context, *grad_output: Tensor) -> Tuple[Optional[Tensor], ...]:  # type: ignore[override]
        prev_stream, next_stream = ctx.prev_stream, ctx.next_stream
        grads: Deque[Tensor] = deque(maxlen=len(grad_output))
        consumed_on = current_stream(get_device(prev_stream))
        with use_stream(prev_stream), use_stream(next_stream):
            for x in reversed(grad_output):
                y = x.to(get_device(prev_stream), non_blocking=True)
                grads.appendleft(y)
                record_stream(x, next_stream)
                record_stream(y, consumed_on)
        return (None, None) + tuple(grads)


class Wait(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Context, prev_stream: AbstractStream, next_stream: AbstractStream, *input: Tensor) -> Tensors:  # type: ignore[override]
        ctx.prev_stream, ctx.next_stream = prev_stream, next_stream
        wait_stream(next_stream, prev_stream)
        return tuple(x.detach() for x in input)

    @staticmethod
    def backward(ctx: Context, *grad_input: Tensor) -> Tuple[Optional[Tensor], ...]:  # type: ignore[override]
        wait_stream(ctx.prev_stream, ctx.next_stream)
        return (None, None) + grad_input
