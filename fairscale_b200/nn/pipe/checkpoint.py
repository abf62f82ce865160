"""Two-node activation checkpointing for pipeline stages.

Parity: fairscale/nn/pipe/checkpoint.py:77-326.  A checkpointed stage contributes two autograd nodes that
share a small mailbox: ``Recompute`` (reached first in backward, because it hangs off the *previous*
micro-batch's output through fork/join) replays the stage with grad enabled and parks the result;
``Checkpoint`` then back-propagates through the parked graph.  Recomputation of micro-batch *i* therefore
overlaps the backward of micro-batch *i+1* on the next stage instead of delaying it.
"""

from __future__ import annotations

import threading
from collections import deque
from contextlib import contextmanager, nullcontext
from typing import Any, Callable, Deque, Generator, List, Optional, Tuple, Union

import torch
from torch import Tensor

from .dependency import fork, join
from .microbatch import Batch
from .phony import get_phony

__all__ = ["is_checkpointing", "is_recomputing"]

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]
Recomputed = Tuple[TensorOrTensors, Tensors]  # (stage output with graph, detached input leaves)
RNGStates = Tuple[Tensor, Optional[Tensor]]
Function = Callable[[TensorOrTensors], TensorOrTensors]


class _Mailbox:
    """What ``Checkpoint`` and ``Recompute`` of one (stage, micro-batch) share."""

    def __init__(self) -> None:
        self.recomputed: Deque[Recomputed] = deque(maxlen=1)
        self.rng_states: Deque[RNGStates] = deque(maxlen=1)
        self.autocast: Optional[dict] = None  # arguments of the autocast context the forward ran under


class Checkpointing:
    """Factory of the ``Checkpoint`` / ``Recompute`` pair for one stage and one micro-batch."""

    def __init__(self, function: Function, batch: Batch) -> None:
        self.function = function
        self.batch = batch
        self._box = _Mailbox()
        # kept for introspection / parity with the reference's attribute names
        self.recomputed = self._box.recomputed
        self.rng_states = self._box.rng_states

    def checkpoint(self) -> Batch:
        """Run the stage without grad; the returned batch carries the ``Checkpoint`` node."""
        atomic = self.batch.atomic
        inputs = tuple(self.batch)
        phony = get_phony(self.batch[0].device, requires_grad=True)  # guarantees the node exists in the graph
        out = Checkpoint.apply(phony, self._box, self.function, atomic, *inputs)
        if isinstance(out, tuple):
            out = tuple(x if x.is_floating_point() else x.detach() for x in out)
        return Batch(out, self.batch.index)

    def recompute(self, batch: Batch) -> None:
        """Attach the ``Recompute`` node to ``batch`` (the stage output) in place."""
        atomic = self.batch.atomic
        inputs = tuple(self.batch)
        batch[0], phony = fork(batch[0])
        phony = Recompute.apply(phony, self._box, self.function, atomic, *inputs)
        batch[0] = join(batch[0], phony)


class _Flags(threading.local):
    def __init__(self) -> None:
        self.is_checkpointing = False
        self.is_recomputing = False


thread_local = _Flags()


@contextmanager
def enable_checkpointing() -> Generator[None, None, None]:
    prev = thread_local.is_checkpointing
    thread_local.is_checkpointing = True
    try:
        yield
    finally:
        thread_local.is_checkpointing = prev


@contextmanager
def enable_recomputing() -> Generator[None, None, None]:
    prev = thread_local.is_recomputing
    thread_local.is_recomputing = True
    try:
        yield
    finally:
        thread_local.is_recomputing = prev


def recomputed_in_backward(function: Callable[[Any], Any], input: Any) -> Any:
    """``function(input)`` through ``torch.utils.checkpoint`` (no activations kept; the call is repeated in backward), with the
    flags of this module raised around the two calls: :func:`is_checkpointing` during the first, :func:`is_recomputing` during
    the repetition, so that layers with side effects (running statistics, counters) can tell them apart.  Used by the
    multi-process pipeline, whose stages checkpoint whole micro-batches."""
    from torch.utils.checkpoint import checkpoint as torch_checkpoint

    calls = [0]

    def flagged(x: Any) -> Any:
        calls[0] += 1
        with (enable_checkpointing() if calls[0] == 1 else enable_recomputing()):
            return function(x)

    return torch_checkpoint(flagged, input, use_reentrant=False)


def is_checkpointing() -> bool:
    """True inside the no-grad forward of a checkpointed stage."""
    return thread_local.is_checkpointing


def is_recomputing() -> bool:
    """True inside the recomputation; guard side effects (counters, running statistics) with it."""
    return thread_local.is_recomputing


def save_rng_states(device: torch.device, rng_states: Deque[RNGStates]) -> None:
    cpu = torch.get_rng_state()
    gpu = torch.cuda.get_rng_state(device) if device.type == "cuda" else None
    rng_states.clear()
    rng_states.append((cpu, gpu))


@contextmanager
def restore_rng_states(device: torch.device, rng_states: Deque[RNGStates]) -> Generator[None, None, None]:
    cpu, gpu = rng_states[0]
    devices: List[torch.device] = [device] if device.type == "cuda" else []
    with torch.random.fork_rng(devices):
        torch.set_rng_state(cpu)
        if gpu is not None:
            torch.cuda.set_rng_state(gpu, device)
        yield


class Checkpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, phony: Tensor, box: _Mailbox, function: Function, input_atomic: bool, *input: Tensor) -> TensorOrTensors:  # type: ignore[override]
        ctx.box = box
        save_rng_states(input[0].device, box.rng_states)
        box.autocast = next(({"device_type": d, "dtype": torch.get_autocast_dtype(d)} for d in ("cuda", "cpu") if torch.is_autocast_enabled(d)), None)
        ctx.save_for_backward(*input)
        with torch.no_grad(), enable_checkpointing():
            return function(input[0] if input_atomic else input)

    @staticmethod
    def backward(ctx: Any, *grad_output: Tensor) -> Tuple[Optional[Tensor], ...]:  # type: ignore[override]
        output, input_leaf = ctx.box.recomputed.pop()
        tensors = output if isinstance(output, tuple) else (output,)
        if any(y.requires_grad for y in tensors):
            pairs = [(y, g) for y, g in zip(tensors, grad_output) if y.requires_grad]
            torch.autograd.backward([y for y, _ in pairs], [g for _, g in pairs])
        return (None, None, None, None) + tuple(x.grad for x in input_leaf)


class Recompute(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, phony: Tensor, box: _Mailbox, function: Function, input_atomic: bool, *input: Tensor) -> Tensor:  # type: ignore[override]
        ctx.box = box
        ctx.function = function
        ctx.input_atomic = input_atomic
        ctx.save_for_backward(*input)
        return phony

    @staticmethod
    def backward(ctx: Any, *grad_output: Tensor) -> Tuple[None, ...]:  # type: ignore[override]
        inputs = ctx.saved_tensors
        leaves = tuple(x.detach().requires_grad_(x.requires_grad) for x in inputs)
        # the repetition runs under the random state and the autocast state of the forward (backward passes start with
        # autocast off, and a stage that got low-precision activations then meets its own fp32 weights)
        amp = torch.autocast(**ctx.box.autocast) if ctx.box.autocast is not None else nullcontext()
        with restore_rng_states(inputs[0].device, ctx.box.rng_states):
            with torch.enable_grad(), enable_recomputing(), amp:
                output = ctx.function(leaves[0] if ctx.input_atomic else leaves)
        ctx.box.recomputed.append((output, leaves))
        return (None, None, None, None) + tuple(None for _ in inputs)
