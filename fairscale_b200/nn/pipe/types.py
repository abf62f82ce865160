"""Shared types of the multi-process pipeline (parity: fairscale/nn/pipe/types.py:13-69)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, List, Optional, Tuple, Union

import torch
from torch import Tensor, nn

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]

MESSAGE_GENERATION_START = 0

# globally unique tag space for p2p messages of one step
_message_generation = MESSAGE_GENERATION_START
MESSAGE_TENSOR_SIZE = 1024  # reserved width of a header; headers here are small fixed int64 tensors


class LazyModule:
    """Deferred construction of a layer so that every rank only builds the layers of its own stage."""

    def __init__(self, function: Callable[[], nn.Module]):
        self.function = function

    def __call__(self) -> nn.Module:
        return self.function()


@dataclass(init=False)
class PipeMessage:
    """Envelope of one activation / gradient transfer between neighbouring stages."""

    src: int
    dest: int
    queue_name: int
    args: Any
    tensors: Tensors
    tensor_shapes: List[torch.Size]
    tensor_dtypes: List[torch.dtype]
    tag: int = 0

    def __init__(self, src: int, dest: int, queue_name: int, args: Any = None, tensors: Optional[Tensors] = None, tensor_count: int = 0):
        self.src = src
        self.dest = dest
        self.queue_name = queue_name
        self.args = args
        self.tensors = tensors or tuple()
        self.tensor_shapes = []
        self.tensor_dtypes = []
        global _message_generation
        self.tag = _message_generation
        _message_generation += len(self.tensors) if tensors is not None else tensor_count
