"""``Pipe``: GPipe for an ``nn.Sequential`` spread over the GPUs of one process.

API parity with fairscale/nn/pipe/pipe.py:174-418: ``Pipe(module, balance, devices=None, chunks=1,
checkpoint="except_last", deferred_batch_norm=False)``, the same validation errors, device-move denial,
``Sequential``-like container protocol.  (The reference's DeprecationWarning is not reproduced.)
"""

from __future__ import annotations

from collections import OrderedDict
from typing import TYPE_CHECKING, Any, Iterable, Iterator, List, Optional, Tuple, Union, cast

import torch
import torch.autograd
import torch.cuda
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

if TYPE_CHECKING:
    Module = nn.Module[TensorOrTensors]
    NamedModules = OrderedDict[str, Module]
else:
    Module = nn.Module
    NamedModules = OrderedDict


def recommend_auto_balance(message: str) -> str:
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
    if len(list(module.named_children())) != len(module):
        raise ValueError("module with duplicate children is not supported")


def verify_splitting(module: nn.Sequential, partitions: List[nn.Sequential], balance: Iterable[int], devices: List[torch.device]) -> None:
    """A parameter shared by layers that ended up on different devices cannot be kept consistent."""
    n_params = len(list(module.parameters()))
    n_child_params = sum(len(list(child.parameters())) for child in module.children())
    if n_params == n_child_params:
        return
    for i in range(len(partitions)):
        for j in range(i + 1, len(partitions)):
            if devices[i] == devices[j]:
                continue
            ids_j = {id(q) for q in partitions[j].parameters()}
            if any(id(p) in ids_j for p in partitions[i].parameters()):
                raise ValueError("module with duplicate parameters on distinct devices is not supported")


class BalanceError(ValueError):
    pass


def split_module(module: nn.Sequential, balance: Iterable[int], devices: List[torch.device]
                 ) -> Tuple[List[nn.Sequential], List[int], List[torch.device]]:
    """Cut ``module`` into consecutive partitions of ``balance`` layers and move each to its device."""
    balance = list(balance)
    if len(module) != sum(balance):
        raise BalanceError(
            f"module and sum of balance have different length (module: {len(module)}, sum of balance: {sum(balance)})"
        )
    if any(x <= 0 for x in balance):
        raise BalanceError(f"all balance numbers must be positive integer (balance: {balance})")
    if len(balance) > len(devices):
        raise IndexError(f"too few devices to hold given partitions (devices: {len(devices)}, partitions: {len(balance)})")

    partitions = []
    layers: NamedModules = OrderedDict()
    j = 0
    for name, layer in module.named_children():
        layers[name] = layer
        if len(layers) == balance[j]:
            partition = nn.Sequential(layers)
            partition.to(devices[j])
            partitions.append(partition)
            layers.clear()
            j += 1
    del devices[j:]
    return cast(List[nn.Sequential], nn.ModuleList(partitions)), balance, devices


MOVING_DENIED = TypeError("denied to move parameters and buffers, because Pipe should manage device placement")


class Pipe(Module):
    """Wrap a sequential model for GPipe training::

        model = Pipe(nn.Sequential(a, b, c, d), balance=[1, 1, 1, 1], chunks=8)
        output = model(input)      # input on the first device, output on the last

    Args:
        module: ``nn.Sequential`` to split.
        balance: layers per partition (``sum(balance) == len(module)``).
        devices: devices to use (default: all CUDA devices, or CPU when there is none).
        chunks: number of micro-batches.
        checkpoint: ``"always"``, ``"except_last"`` (default) or ``"never"``.
        deferred_batch_norm: accumulate BatchNorm statistics over the whole mini-batch.
    """

    balance: List[int] = []
    devices: List[torch.device] = []
    chunks: int = 1
    checkpoint: str = "except_last"

    def __init__(self, module: nn.Sequential, balance: Optional[Iterable[int]] = None, *, devices: Optional[Devices] = None,
                 chunks: int = chunks, checkpoint: str = checkpoint, deferred_batch_norm: bool = False) -> None:
        super().__init__()
        chunks = int(chunks)
        checkpoint = str(checkpoint)
        if balance is None:
            raise ValueError(recommend_auto_balance("balance is required"))
        if chunks <= 0:
            raise ValueError("number of chunks must be positive integer")
        if checkpoint not in ["always", "except_last", "never"]:
            raise ValueError("checkpoint is not one of 'always', 'except_last', or 'never'")

        verify_module(module)
        verify_skippables(module)  # TypeError for unmatched stash / pop pairs

        self.chunks = chunks
        self.checkpoint = checkpoint
        if deferred_batch_norm:
            module = DeferredBatchNorm.convert_deferred_batch_norm(module, chunks)

        if devices is None:
            devices = range(torch.cuda.device_count()) if torch.cuda.is_available() else ["cpu"] * len(list(balance))
        devices = [torch.device(d) for d in devices]
        devices = cast(List[torch.device], devices)
        try:
            self.partitions, self.balance, self.devices = split_module(module, balance, devices)
        except BalanceError as exc:
            raise ValueError(recommend_auto_balance(str(exc)))
        verify_splitting(module, self.partitions, self.balance, self.devices)

        self._copy_streams: List[List[AbstractStream]] = []
        self._skip_layout = inspect_skip_layout(self.partitions)
        checkpoint_stop = {"always": self.chunks, "except_last": self.chunks - 1, "never": 0}[self.checkpoint]
        self.pipeline = Pipeline(self.partitions, self.devices, self._ensure_copy_streams(), self._skip_layout, checkpoint_stop)

    # ------------------------------------------------------------------ Sequential-like protocol
    def __len__(self) -> int:
        return sum(len(p) for p in self.partitions)

    def __getitem__(self, index: int) -> nn.Module:
        partitions = self.partitions
        if index < 0:
            partitions = partitions[::-1]
        for partition in partitions:
            try:
                return partition[index]
            except IndexError:
                pass
            shift = len(partition)
            index = index + shift if index < 0 else index - shift
        raise IndexError

    def __iter__(self) -> Iterable[nn.Module]:
        for partition in self.partitions:
            yield from partition

    # ------------------------------------------------------------------ device placement is Pipe's business
    def cuda(self, device: Optional[Device] = None) -> "Pipe":
        raise MOVING_DENIED

    def cpu(self) -> "Pipe":
        raise MOVING_DENIED

    def to(self, *args: Any, **kwargs: Any) -> "Pipe":
        """Only dtype conversions are allowed."""
        if "device" in kwargs or "tensor" in kwargs:
            raise MOVING_DENIED
        if args and isinstance(args[0], (torch.device, int, str, torch.Tensor)):
            raise MOVING_DENIED
        return super().to(*args, **kwargs)

    def _ensure_copy_streams(self) -> List[List[AbstractStream]]:
        """One copy stream per (partition, micro-batch) so copies of different micro-batches overlap."""
        if not self._copy_streams:
            for device in self.devices:
                self._copy_streams.append([new_stream(device) for _ in range(self.chunks)])
        return self._copy_streams

    def forward(self, input: TensorOrTensors) -> TensorOrTensors:  # type: ignore[override]
        microbatch.check(input)
        if not self.devices:
            return input  # an empty sequential module
        batches = microbatch.scatter(input, self.chunks)
        self.pipeline.run(batches)
        return microbatch.gather(batches)
