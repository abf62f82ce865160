"""Uniform handling of CUDA streams and the CPU "stream" placeholder (parity: fairscale/nn/pipe/stream.py:31-134)."""

from __future__ import annotations

from contextlib import contextmanager
from typing import Generator, List, Union, cast

import torch

__all__: List[str] = []


class CPUStreamType:
    pass


CPUStream = CPUStreamType()
AbstractStream = Union[torch.cuda.Stream, CPUStreamType]


def new_stream(device: torch.device) -> AbstractStream:
    return CPUStream if device.type != "cuda" else torch.cuda.Stream(device)


def current_stream(device: torch.device) -> AbstractStream:
    return CPUStream if device.type != "cuda" else torch.cuda.current_stream(device)


def default_stream(device: torch.device) -> AbstractStream:
    return CPUStream if device.type != "cuda" else torch.cuda.default_stream(device)


@contextmanager
def use_device(device: torch.device) -> Generator[None, None, None]:
    if device.type != "cuda":
        yield
        return
    with torch.cuda.device(device):
        yield


@contextmanager
def use_stream(stream: AbstractStream) -> Generator[None, None, None]:
    if not is_cuda(stream):
        yield
        return
    with torch.cuda.stream(as_cuda(stream)):
        yield


def get_device(stream: AbstractStream) -> torch.device:
    return as_cuda(stream).device if is_cuda(stream) else torch.device("cpu")


def wait_stream(source: AbstractStream, target: AbstractStream) -> None:
    """``source`` waits for the work currently queued on ``target``."""
    if is_cuda(target):
        if is_cuda(source):
            as_cuda(source).wait_stream(as_cuda(target))
        else:
            as_cuda(target).synchronize()  # the CPU waits for the device
    # a CUDA stream never needs to wait for the (synchronous) CPU


def record_stream(tensor: torch.Tensor, stream: AbstractStream) -> None:
    """Tell the caching allocator that ``tensor`` is in use on ``stream``."""
    if is_cuda(stream) and tensor.is_cuda:
        # record on a view of the whole storage so that shifted views are covered too
        tensor = tensor.new_empty([0]).set_(tensor.untyped_storage())
        tensor.record_stream(as_cuda(stream))


def is_cuda(stream: AbstractStream) -> bool:
    return stream is not CPUStream


def as_cuda(stream: AbstractStream) -> torch.cuda.Stream:
    return cast(torch.cuda.Stream, stream)
