"""Mini-batch <-> micro-batch conversion (parity: fairscale/nn/pipe/microbatch.py:36-203)."""

from __future__ import annotations

import typing
from typing import Any, Callable, Iterable, Iterator, List, Tuple, Union, cast

import torch
from torch import Tensor

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]
Function = Callable[[TensorOrTensors], TensorOrTensors]


class Batch:
    """A micro-batch: one tensor or a tuple of tensors, with uniform access helpers."""

    def __init__(self, value: TensorOrTensors, index: int) -> None:
        self.value = value
        self.atomic = torch.is_tensor(value)
        self.__index = index

    @property
    def index(self) -> int:
        return self.__index

    @property
    def tensor(self) -> Tensor:
        if not self.atomic:
            raise AttributeError("not atomic batch")
        return cast(Tensor, self.value)

    @property
    def tensors(self) -> Tensors:
        if self.atomic:
            raise AttributeError("batch is atomic")
        return cast(Tensors, self.value)

    @property
    def tensor_or_tensors(self) -> TensorOrTensors:
        return self.value

    def call(self, function: Function) -> "Batch":
        return Batch(function(self.value), self.index)

    def __repr__(self) -> str:
        return f"Batch[atomic={self.atomic!r}]({self.value!r})"

    def __iter__(self) -> Iterator[Tensor]:
        if self.atomic:
            yield self.tensor
        else:
            yield from self.tensors

    def __len__(self) -> int:
        return 1 if self.atomic else len(self.tensors)

    def __getitem__(self, index: int) -> Tensor:
        if not self.atomic:
            return self.tensors[index]
        if index != 0:
            raise IndexError("atomic batch allows index 0 only")
        return self.tensor

    def __setitem__(self, index: Union[int, slice], value: Any) -> None:
        if isinstance(index, int):
            if self.atomic:
                if index != 0:
                    raise IndexError("atomic batch allows index 0 only")
                self.value = value
            else:
                self.value = self.tensors[:index] + (value,) + self.tensors[index + 1:]
            return
        if not (index.start is index.stop is index.step is None):
            raise NotImplementedError("only slice [:] supported")
        if not self.atomic:
            self.value = tuple(value)
            return
        if len(value) != 1:
            raise IndexError("atomic batch cannot be replaced with multiple tensors")
        self.value = value[0]


def check(input: TensorOrTensors) -> None:
    """Inputs / outputs of a pipeline must be a tensor or a tuple of tensors."""
    if isinstance(input, tuple):
        for x in input:
            check(x)
        return
    if not isinstance(input, Tensor):
        raise TypeError(f"expected Tensor, but got {input.__class__.__name__}")


def scatter(input: TensorOrTensors, chunks: int) -> List[Batch]:
    """Split along dim 0 into at most ``chunks`` micro-batches (``Tensor.chunk`` semantics)."""
    if isinstance(input, Tensor):
        pieces: Iterable[TensorOrTensors] = input.chunk(chunks)
    else:
        per_tensor = [t.chunk(chunks) for t in input]
        pieces = zip(*per_tensor)
    return [Batch(x, i) for i, x in enumerate(pieces)]


def gather(outputs: List[Batch]) -> TensorOrTensors:
    """Concatenate micro-batch outputs along dim 0."""
    if outputs[0].atomic:
        return torch.cat(tuple(b.tensor for b in outputs))
    columns = zip(*(b.tensors for b in outputs))
    return tuple(torch.cat(col) for col in columns)
