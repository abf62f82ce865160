"""Shared types of the multi-process pipeline (names of fairscale/nn/pipe/types.py:13-69)."""

from __future__ import annotations

from typing import Any, Callable, List, Optional, Tuple, Union

import torch
from torch import Tensor, nn

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]

MESSAGE_GENERATION_START = 0
MESSAGE_TENSOR_SIZE = 1024  # reserved width of a header; headers here are small fixed int64 tensors


class _TagSpace:
    """Tags of p2p messages, unique within the process: every message reserves one tag per tensor it carries."""

    def __init__(self, start: int) -> None:
        self.next = start

    def reserve(self, count: int) -> int:
        first, self.next = self.next, self.next + count
        return first


_tags = _TagSpace(MESSAGE_GENERATION_START)


class LazyModule:
    """Deferred construction of a layer so that every rank only builds the layers of its own stage."""

    def __init__(self, function: Callable[[], nn.Module]):
        self.function = function

    def __call__(self) -> nn.Module:
        return self.function()


class PipeMessage:
    """Envelope of one activation / gradient transfer between neighbouring stages: who sends to whom, which queue of the
    receiver it is for, small Python arguments, and the tensors (whose shapes and dtypes the sender fills in)."""

    __slots__ = ("src", "dest", "queue_name", "args", "tensors", "tensor_shapes", "tensor_dtypes", "tag")

    def __init__(self, src: int, dest: int, queue_name: int, args: Any = None, tensors: Optional[Tensors] = None, tensor_count: int = 0):
        self.src, self.dest, self.queue_name, self.args = src, dest, queue_name, args
        self.tensors: Tensors = tuple(tensors) if tensors else tuple()
        self.tensor_shapes: List[torch.Size] = []
        self.tensor_dtypes: List[torch.dtype] = []
        self.tag = _tags.reserve(len(self.tensors) if tensors is not None else tensor_count)

    def __repr__(self) -> str:
        return f"PipeMessage({self.src}->{self.dest}, queue {self.queue_name}, {len(self.tensors)} tensors, tag {self.tag})"


