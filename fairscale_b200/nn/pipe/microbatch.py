"""Micro-batches: the unit of work that moves through a pipeline.

A :class:`Batch` is either *atomic* (it wraps one tensor, and modules see that tensor) or a tuple of tensors (modules
see the tuple).  ``scatter`` cuts a mini-batch along dimension 0, ``gather`` concatenates the results again.
Contract of fairscale/nn/pipe/microbatch.py:36-203.
"""

from __future__ import annotations

from typing import Callable, Iterable, Iterator, List, Tuple, Union, cast

import torch
from torch import Tensor

__all__: List[str] = []

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]
Function = Callable[[TensorOrTensors], TensorOrTensors]


class Batch:
    """Holds the tensors of one micro-batch plus its position ``index`` in the mini-batch."""

    __slots__ = ("_items", "atomic", "_index")

    def __init__(self, value: TensorOrTensors, index: int) -> None:
        self.atomic = torch.is_tensor(value)
        self._items: List[Tensor] = [cast(Tensor, value)] if self.atomic else list(cast(Tensors, value))
        self._index = index

    # -- views of the payload
    @property
    def index(self) -> int:
        return self._index

    @property
    def tensor(self) -> Tensor:
        if not self.atomic:
            raise AttributeError("not atomic batch")
        return self._items[0]

    @property
    def tensors(self) -> Tensors:
        if self.atomic:
            raise AttributeError("batch is atomic")
        return tuple(self._items)

    @property
    def tensor_or_tensors(self) -> TensorOrTensors:
        return self._items[0] if self.atomic else tuple(self._items)

    def call(self, function: Function) -> "Batch":
        """``function`` applied to the payload, wrapped as a batch with the same index."""
        return Batch(function(self.tensor_or_tensors), self._index)

    # -- list protocol over the tensors (an atomic batch has length 1)
    def __repr__(self) -> str:
        return f"Batch[{self._index}, atomic={self.atomic}]({self.tensor_or_tensors!r})"

    def __len__(self) -> int:
        return len(self._items)

    def __iter__(self) -> Iterator[Tensor]:
        return iter(self._items)

    def __getitem__(self, key):  # type: ignore[no-untyped-def]
        picked = self._items[key]
        return tuple(picked) if isinstance(key, slice) else picked

    def __setitem__(self, key, value) -> None:  # type: ignore[no-untyped-def]
        if isinstance(key, slice):
            new_items = list(self._items)
            new_items[key] = list(value)
            if self.atomic and len(new_items) != 1:
                raise ValueError("an atomic batch holds exactly one tensor")
            self._items = new_items
        else:
            self._items[key] = value


def check(input: TensorOrTensors) -> None:
    """``TypeError`` unless ``input`` is a tensor or a tuple of tensors."""
    if torch.is_tensor(input):
        return
    if not isinstance(input, tuple):
        raise TypeError(f"expected Tensor or Tensors, but got {type(input).__name__}")
    for member in input:
        if not torch.is_tensor(member):
            raise TypeError(f"expected Tensor, but got {type(member).__name__}")


def scatter(input: TensorOrTensors, chunks: int) -> List[Batch]:
    """Cut ``input`` into at most ``chunks`` micro-batches along dimension 0 (fewer when the batch is small)."""
    if torch.is_tensor(input):
        pieces: Iterable[TensorOrTensors] = cast(Tensor, input).chunk(chunks)
    else:
        columns = [t.chunk(chunks) for t in cast(Tensors, input)]  # per tensor: its pieces
        pieces = zip(*columns)                                      # per micro-batch: one piece of every tensor
    return [Batch(piece, i) for i, piece in enumerate(pieces)]


def gather(outputs: List[Batch]) -> TensorOrTensors:
    """Concatenate the micro-batches back into one mini-batch."""
    if outputs[0].atomic:
        return torch.cat([b.tensor for b in outputs])
    rows = [b.tensors for b in outputs]
    return tuple(torch.cat(column) for column in zip(*rows))
