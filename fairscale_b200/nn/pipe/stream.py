"""One vocabulary for CUDA streams and "the CPU stream", so that the pipeline code has no device-type branches.

Function names and meanings follow fairscale/nn/pipe/stream.py:24-123.  A CPU "stream" is the singleton
:data:`CPUStream`; every operation on it is a no-op (CPU work is synchronous).
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Generator, List, Union

import torch

__all__: List[str] = []


class CPUStreamType:
    def __repr__(self) -> str:
        return "CPUStream"


CPUStream = CPUStreamType()
AbstractStream = Union[torch.cuda.Stream, CPUStreamType]


def is_cuda(stream: AbstractStream) -> bool:
    return not isinstance(stream, CPUStreamType)


def as_cuda(stream: AbstractStream) -> torch.cuda.Stream:
    assert is_cuda(stream), "a CUDA stream is required here"
    return stream  # type: ignore[return-value]


def _pick(device: torch.device, cuda_factory) -> AbstractStream:  # type: ignore[no-untyped-def]
    return cuda_factory(device) if torch.device(device).type == "cuda" else CPUStream


def new_stream(device: torch.device) -> AbstractStream:
    return _pick(device, torch.cuda.Stream)


def current_stream(device: torch.device) -> AbstractStream:
    return _pick(device, torch.cuda.current_stream)


def default_stream(device: torch.device) -> AbstractStream:
    return _pick(device, torch.cuda.default_stream)


def get_device(stream: AbstractStream) -> torch.device:
    return as_cuda(stream).device if is_cuda(stream) else torch.device("cpu")


@contextmanager
def use_device(device: torch.device) -> Generator[None, None, None]:
    if torch.device(device).type == "cuda":
        with torch.cuda.device(device):
            yield
    else:
        yield


@contextmanager
def use_stream(stream: AbstractStream) -> Generator[None, None, None]:
    if is_cuda(stream):
        with torch.cuda.stream(as_cuda(stream)):
            yield
    else:
        yield


def wait_stream(source: AbstractStream, target: AbstractStream) -> None:
    """Work queued on ``source`` after this call starts only when what is queued on ``target`` now has finished."""
    if not is_cuda(target):
        return
    if is_cuda(source):
        as_cuda(source).wait_stream(as_cuda(target))
    else:
        as_cuda(target).synchronize()  # the host itself is the waiter


def record_stream(tensor: torch.Tensor, stream: AbstractStream) -> None:
    """Tell the caching allocator that ``tensor`` is in use on ``stream`` (its block is not recycled before)."""
    if not is_cuda(stream):
        return
    tensor.record_stream(as_cuda(stream))
