"""``Pipe``: GPipe for an ``nn.Sequential`` whose layers are spread over the devices of one process.

    model = Pipe(nn.Sequential(a, b, c, d), balance=[2, 2], devices=[0, 1], chunks=8)
    output = model(input)            # input on the first device, output on the last

The constructor validates the arguments, cuts the sequential module into one partition per entry of ``balance`` and
moves each partition to its device; ``forward`` splits the mini-batch into ``chunks`` micro-batches and hands them to
the executor in ``pipeline.py``.  Constructor signature, error types and messages, the refusal to move the wrapped
module and the ``Sequential``-like container protocol follow fairscale/nn/pipe/pipe.py:75-418 (its deprecation warning is
not reproduced).
"""

from __future__ import annotations

from typing import Any, Iterable, Iterator, List, Optional, Sequence, Tuple, Union

import torch
from torch import Tensor, nn

from . import microbatch
from .batchnorm import DeferredBatchNorm
from .pipeline import Pipeline
from .skip.layout import inspect_skip_layout
from .skip.skippable import verify_skippables
from .stream import AbstractStream, new_stream

__all__ = ["Pipe"]

Device = Union[torch.device, int, str]
Devices = Union[Iterable[Device], List[Device]]
Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]

_CHECKPOINT_MODES = ("always", "except_last", "never")


class BalanceError(ValueError):
    """The layer counts in ``balance`` do not describe the module."""


def recommend_auto_balance(message: str) -> str:
    """``message`` followed by a pointer to the automatic balancing helpers."""
    return f"""{message}

If your model is still under development, its optimal balance would change
frequently. In this case, we highly recommend 'fairscale_b200.nn.pipe.balance' for
naive automatic balancing:

  from fairscale_b200.nn import Pipe
  from fairscale_b200.nn.pipe.balance import balance_by_time

  partitions = torch.cuda.device_count()
  sample = torch.empty(...)
  balance = balance_by_time(partitions, model, sample)

  model = Pipe(model, balance, ...)
"""


def verify_module(module: nn.Sequential) -> None:
    if not isinstance(module, nn.Sequential):
        raise TypeError("module must be nn.Sequential to be partitioned")
    children = list(module.children())  # children() de-duplicates
    if len(children) != len(module):
        raise ValueError("module with duplicate children is not supported")


def verify_splitting(module: nn.Sequential, partitions: Sequence[nn.Sequential], balance: Iterable[int],
                     devices: Sequence[torch.device]) -> None:
    """A parameter that two layers share must not end up on two devices: its copies could not be kept equal."""
    owner: dict = {}  # id(parameter) -> device of the partition that was seen holding it first
    for partition, device in zip(partitions, devices):
        for p in partition.parameters():
            if owner.setdefault(id(p), device) != device:
                raise ValueError("module with duplicate parameters on distinct devices is not supported")


def split_module(module: nn.Sequential, balance: Iterable[int], devices: List[torch.device]
                 ) -> Tuple[List[nn.Sequential], List[int], List[torch.device]]:
    """Partitions of ``balance[k]`` consecutive layers each, every one moved to ``devices[k]``.  Returns the partitions
    (registered in a ``ModuleList``), the balance as a list and the devices actually used."""
    balance = list(balance)
    if sum(balance) != len(module):
        raise BalanceError(f"module and sum of balance have different length (module: {len(module)}, sum of balance: {sum(balance)})")
    if min(balance, default=1) <= 0:
        raise BalanceError(f"all balance numbers must be positive integer (balance: {balance})")
    if len(devices) < len(balance):
        raise IndexError(f"too few devices to hold given partitions (devices: {len(devices)}, partitions: {len(balance)})")

    named = list(module.named_children())
    partitions: List[nn.Sequential] = []
    start = 0
    for count, device in zip(balance, devices):
        part = nn.Sequential()
        for name, layer in named[start:start + count]:
            part.add_module(name, layer)  # layers keep their names, so state-dict keys only gain the partition index
        partitions.append(part.to(device))
        start += count
    return nn.ModuleList(partitions), balance, list(devices[: len(balance)])  # type: ignore[return-value]


def _moving_denied() -> TypeError:
    return TypeError("denied to move parameters and buffers, because Pipe should manage device placement")


class Pipe(nn.Module):
    """See the module docstring.

    Args:
        module: the ``nn.Sequential`` to pipeline.
        balance: number of layers per partition; its sum must be ``len(module)``.
        devices: one device per partition (default: the CUDA devices in order, or CPU if there is none).
        chunks: number of micro-batches a mini-batch is cut into.
        checkpoint: which micro-batches recompute their forward in backward - ``"always"``, ``"except_last"``
            (all but the last micro-batch, whose backward starts right after its forward) or ``"never"``.
        deferred_batch_norm: let BatchNorm layers track running statistics per mini-batch (``batchnorm.py``).
    """

    balance: List[int] = []
    devices: List[torch.device] = []
    chunks: int = 1
    checkpoint: str = "except_last"

    def __init__(self, module: nn.Sequential, balance: Optional[Iterable[int]] = None, *, devices: Optional[Devices] = None,
                 chunks: int = chunks, checkpoint: str = checkpoint, deferred_batch_norm: bool = False) -> None:
        super().__init__()
        chunks, checkpoint = int(chunks), str(checkpoint)
        if balance is None:
            raise ValueError(recommend_auto_balance("balance is required"))
        if chunks <= 0:
            raise ValueError("number of chunks must be positive integer")
        if checkpoint not in _CHECKPOINT_MODES:
            raise ValueError("checkpoint is not one of 'always', 'except_last', or 'never'")
        verify_module(module)
        verify_skippables(module)  # TypeError when stash / pop declarations do not pair up

        self.chunks, self.checkpoint = chunks, checkpoint
        if deferred_batch_norm:
            module = DeferredBatchNorm.convert_deferred_batch_norm(module, chunks)

        balance = list(balance)
        if devices is None:
            devices = range(torch.cuda.device_count()) if torch.cuda.is_available() else ["cpu"] * len(balance)
        try:
            self.partitions, self.balance, self.devices = split_module(module, balance, [torch.device(d) for d in devices])
        except BalanceError as exc:
            raise ValueError(recommend_auto_balance(str(exc))) from None
        verify_splitting(module, self.partitions, self.balance, self.devices)

        # one copy stream per (partition, micro-batch): transfers of different micro-batches overlap each other and compute
        self._copy_streams: List[List[AbstractStream]] = [[new_stream(d) for _ in range(chunks)] for d in self.devices]
        self._skip_layout = inspect_skip_layout(self.partitions)
        recomputed = {"always": chunks, "except_last": chunks - 1, "never": 0}[checkpoint]  # micro-batches [0, recomputed)
        self.pipeline = Pipeline(self.partitions, self.devices, self._copy_streams, self._skip_layout, recomputed)

    # ------------------------------------------------------------------ the layers, as nn.Sequential exposes them
    def _layers(self) -> List[nn.Module]:
        return [layer for partition in self.partitions for layer in partition]

    def __len__(self) -> int:
        return len(self._layers())

    def __iter__(self) -> Iterator[nn.Module]:
        return iter(self._layers())

    def __getitem__(self, index: int) -> nn.Module:
        layers = self._layers()
        if not -len(layers) <= index < len(layers):
            raise IndexError
        return layers[index]

    # ------------------------------------------------------------------ devices are fixed at construction
    def cuda(self, device: Optional[Device] = None) -> "Pipe":
        raise _moving_denied()

    def cpu(self) -> "Pipe":
        raise _moving_denied()

    def to(self, *args: Any, **kwargs: Any) -> "Pipe":
        """dtype conversions pass through; anything that names a device or a tensor to follow is refused."""
        names_device = bool(args) and isinstance(args[0], (torch.device, int, str, torch.Tensor))
        if names_device or "device" in kwargs or "tensor" in kwargs:
            raise _moving_denied()
        return super().to(*args, **kwargs)

    # ------------------------------------------------------------------ running
    def forward(self, input: TensorOrTensors) -> TensorOrTensors:  # type: ignore[override]
        """``input`` (a tensor or tuple of tensors on the first device) through all partitions; the result lives on
        the last device.  Batches smaller than ``chunks`` simply give fewer micro-batches."""
        microbatch.check(input)
        if not self.devices:
            return input  # nothing to run: an empty sequential module
        batches = microbatch.scatter(input, self.chunks)
        self.pipeline.run(batches)
        return microbatch.gather(batches)
