"""Event-driven schedule of the multi-process pipeline, including layers that are called more than once.

Capability parity with fairscale/nn/pipe/async_schedule.py:38-511 (``Location``, ``Invocation``, ``ModuleWrapper``,
``AsyncRecvOperator``, ``AutogradWithoutActivations``, ``AsyncEventLoop`` with its head / middle / tail roles).

A sequential model is a list of *invocations*; invocation ``k`` runs the layer stored at ``Location(stage, index)``.
When the same layer object appears twice in the ``nn.Sequential`` (weight sharing), both invocations run on the stage
that owns the layer, so data may travel back and forth between stages.  Every rank walks its own events
``(invocation, micro-batch)`` in one global order, the wavefront ``order + micro_batch`` and then ``order``: an event's
input is produced by an event that is earlier in that order, sends are asynchronous and receives blocking, so the earliest
unfinished event of the whole pipeline can always run (no deadlock), and the messages between any two ranks are sent
and received in the same sequence (no tags needed, which NCCL does not have).

The loop keeps no activation alive after it has been sent: ``AutogradWithoutActivations`` leaves a one-element stand-in
connected to the graph, and backward feeds the gradient that comes back from the consumer through it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
from torch import Tensor, nn

from .messages import SendRecvTransport


@dataclass(frozen=True)
class Location:
    """Where a layer lives: pipeline stage (group rank) and position among that stage's layers."""

    stage: int
    index: int

    def __repr__(self) -> str:
        return f"{self.stage}@{self.index}"


@dataclass
class Invocation:
    """The ``order``-th call of the sequential model: run ``this``, fed by ``source`` (None: the pipeline input),
    feeding ``dest`` (None: the pipeline output)."""

    order: int
    this: Location
    source: Optional[Location]
    dest: Optional[Location]


@dataclass
class ModuleWrapper:
    """A layer (or a fused run of layers) of one stage with every invocation that executes it."""

    module: nn.Sequential
    location: Location
    invocations: List[Invocation] = field(default_factory=list)


class AsyncRecvOperator(torch.autograd.Function):
    """Receives the activation of an event from ``src_rank``; its backward ships the gradient back there."""

    @staticmethod
    def forward(ctx: Any, phony: Tensor, transport: SendRecvTransport, src_rank: int) -> Tensor:  # type: ignore[override]
        ctx.transport, ctx.src_rank = transport, src_rank
        out = transport.recv(src_rank)
        wants_grad = out.requires_grad  # the sender's flag, carried in the message header
        out = out.detach()
        if not wants_grad or not out.is_floating_point():
            ctx.mark_non_differentiable(out)  # the sender does not wait for a gradient either
        return out

    @staticmethod
    def backward(ctx: Any, grad: Tensor) -> Tuple[Optional[Tensor], ...]:  # type: ignore[override]
        ctx.transport.send(grad, ctx.src_rank)
        return None, None, None


class AutogradWithoutActivations(torch.autograd.Function):
    """One-element stand-in for an activation that has left the stage.  ``backward`` returns ``grad_from_pipeline``
    (set on the graph node when the consumer's gradient arrives) as the gradient of the real activation, so the
    activation tensor itself need not be kept."""

    @staticmethod
    def forward(ctx: Any, *x: Tensor) -> Tensor:  # type: ignore[override]
        return torch.zeros(1, device=x[0].device)

    @staticmethod
    def backward(ctx: Any, grad: Tensor) -> Tuple[Tensor, ...]:  # type: ignore[override]
        assert getattr(ctx, "grad_from_pipeline", None) is not None, "gradient from the next stage was not attached"
        return ctx.grad_from_pipeline


class AsyncEventLoop:
    """Runs the events of one rank for one mini-batch (forward), then the matching backward.

    ``partitions`` are this rank's layers; together their invocations are this rank's share of the model.  The rank
    that owns invocation 0 is the *head* (it consumes the input micro-batches), the owner of the last invocation the
    *tail* (it returns the outputs); every other rank only relays.  A rank can be head and tail at once.
    """

    def __init__(self, partitions: List[ModuleWrapper], rank: int, transport: SendRecvTransport, checkpoint_stop: int = 0):
        self.partitions = partitions
        self.rank = rank
        self.transport = transport
        self.checkpoint_stop = checkpoint_stop
        self._mine: List[Tuple[Invocation, ModuleWrapper]] = sorted(
            ((inv, w) for w in partitions for inv in w.invocations), key=lambda iw: iw[0].order
        )
        self._awaiting_grad: List[Tuple[int, Tensor]] = []  # (consumer stage, stand-in) in the order of the sends

    # ------------------------------------------------------------------ roles
    @property
    def is_head(self) -> bool:
        return any(inv.source is None for inv, _ in self._mine)

    @property
    def is_tail(self) -> bool:
        return any(inv.dest is None for inv, _ in self._mine)

    def _events(self, chunks: int) -> List[Tuple[Invocation, ModuleWrapper, int]]:
        ev = [(inv, w, mb) for inv, w in self._mine for mb in range(chunks)]
        ev.sort(key=lambda e: (e[0].order + e[2], e[0].order))
        return ev

    def _run_module(self, w: ModuleWrapper, x: Tensor, mb: int) -> Tensor:
        if mb < self.checkpoint_stop and torch.is_grad_enabled() and x.requires_grad:
            from .checkpoint import recomputed_in_backward

            return recomputed_in_backward(w.module, x)
        return w.module(x)

    # ------------------------------------------------------------------ forward
    def run_forward(self, batches: Optional[List[Tensor]], chunks: int) -> Optional[List[Tensor]]:
        """All events of this rank for ``chunks`` micro-batches; returns the outputs on the tail, ``None`` elsewhere."""
        local: Dict[Tuple[int, int], Tensor] = {}
        outputs: List[Optional[Tensor]] = [None] * chunks
        self._awaiting_grad = []
        for inv, w, mb in self._events(chunks):
            if inv.source is None:
                assert batches is not None, "the head rank needs the input micro-batches"
                x = batches[mb]
            elif inv.source.stage == self.rank:
                x = local.pop((inv.order - 1, mb))
            else:
                phony = torch.empty(0, device=self.transport.device, requires_grad=torch.is_grad_enabled())
                x = AsyncRecvOperator.apply(phony, self.transport, inv.source.stage)
            y = self._run_module(w, x, mb)
            assert isinstance(y, Tensor), "stages of the multi-process pipeline exchange single tensors"
            if inv.dest is None:
                outputs[mb] = y
            elif inv.dest.stage == self.rank:
                local[(inv.order, mb)] = y
            else:
                self.transport.send(y, inv.dest.stage)
                if y.requires_grad:
                    self._awaiting_grad.append((inv.dest.stage, AutogradWithoutActivations.apply(y)))
        assert not local, "an activation was produced for a local consumer that never ran"
        self.transport.flush()  # every send of the forward pass has been matched before backward reuses the channel
        return outputs if self.is_tail else None  # type: ignore[return-value]

    # the reference names the three shapes of the loop; here they are views of the same event walk
    def event_loop_head(self, batches: List[Tensor], chunks: int) -> Optional[List[Tensor]]:
        assert self.is_head
        return self.run_forward(batches, chunks)

    def event_loop_tail(self, chunks: int) -> List[Tensor]:
        assert self.is_tail
        out = self.run_forward(None, chunks)
        assert out is not None
        return out

    def event_loop(self, chunks: int) -> None:
        assert not self.is_head and not self.is_tail
        self.run_forward(None, chunks)

    # ------------------------------------------------------------------ backward
    def run_backward(self) -> None:
        """Receive the gradient of every activation this rank sent away, newest first, and back-propagate it.  On the
        tail this runs after the user's ``loss.backward()``."""
        for consumer, stand_in in reversed(self._awaiting_grad):
            grad = self.transport.recv(consumer)
            stand_in.grad_fn.grad_from_pipeline = (grad,)  # type: ignore[union-attr]
            torch.autograd.backward(stand_in, torch.ones_like(stand_in))
        self._awaiting_grad = []
        self.transport.flush()
