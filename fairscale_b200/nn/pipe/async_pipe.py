"""Multi-process pipeline: one stage per rank, activations and gradients over NCCL / gloo p2p.

Capability parity with fairscale/nn/pipe/async_pipe.py:65-401 (``AsyncPipe(module, balance, group=...,
chunks=..., checkpoint=...)``, lazy per-rank construction with ``LazyModule``, idle ranks beyond
``len(balance)``, ``back_helper`` on non-final stages).  The schedule is GPipe's: a stage forwards its
micro-batches in order as they arrive and backwards them in reverse; sends are asynchronous so a stage
computes micro-batch *i+1* while micro-batch *i* is on the wire.
"""

from __future__ import annotations

import logging
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Iterable, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor, nn

from . import microbatch
from .async_pipeline import AsyncPipeline
from .async_schedule import Invocation, Location, ModuleWrapper
from .batchnorm import DeferredBatchNorm
from .messages import SendRecvTransport, get_transport
from .skip.skippable import Skippable
from .types import LazyModule

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]


class _RecvBoundary(torch.autograd.Function):
    """Identity on a received activation whose backward ships the gradient to the previous stage."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, transport: SendRecvTransport, prev_rank: int, slot: Optional[int] = None) -> Tensor:  # type: ignore[override]
        ctx.transport, ctx.prev_rank, ctx.slot = transport, prev_rank, slot
        return x.view_as(x)

    @staticmethod
    def backward(ctx: Any, grad: Tensor):  # type: ignore[override]
        ctx.transport.send(grad, ctx.prev_rank, slot=ctx.slot)
        return grad, None, None, None


def check_balance(module: Union[nn.Sequential, List[LazyModule]], balance: Sequence[int]) -> None:
    if len(module) != sum(balance):
        raise ValueError(f"module and sum of balance have different length (module: {len(module)}, sum of balance: {sum(balance)})")
    if any(x <= 0 for x in balance):
        raise ValueError(f"all balance numbers must be positive integer (balance: {list(balance)})")


def verify_module(module: Union[nn.Sequential, List[LazyModule]]) -> None:
    """The reference refuses a layer object that occurs twice in a plain :class:`Pipe`; ``AsyncPipe`` here accepts it and
    switches to the event-loop schedule, so this check only serves callers that want the strict behaviour."""
    if len(set(map(id, module))) != len(module):
        raise ValueError("module with duplicate children is not supported")


@dataclass
class PartitionInfo:
    """Layers of one location (name -> module) and the invocations that run them."""

    location: Location
    modules: "OrderedDict[str, nn.Module]"
    invocations: List[Invocation] = field(default_factory=list)

    def __len__(self) -> int:
        return len(self.modules)


def _refuse_lazy_skippables(module: Any, layers: Iterable[nn.Module]) -> None:
    """Skip connections are resolved against the whole sequence, which a rank that only builds its own layers never sees."""
    if not isinstance(module, nn.Sequential) and any(isinstance(layer, Skippable) for layer in layers):
        raise ValueError("Can't use Skippable layers with multi-process pipe and lazy construction")


def plan_invocations(layers: Sequence[Any], balance: Sequence[int]) -> Tuple[List[Location], List[Invocation]]:
    """Where every entry of the layer list runs, and the chain of invocations.

    Entry ``i`` nominally belongs to the stage given by ``balance``; an entry that is the same object as an earlier one
    (a shared layer) runs where its first occurrence lives.  Returns one ``Location`` per entry and one ``Invocation``
    per entry (parity: ``instantiate_partition`` in fairscale/nn/pipe/async_pipe.py:224-319)."""
    first: dict = {}
    per_stage_count = [0] * len(balance)
    locations: List[Location] = []
    stage, used = 0, 0
    for layer in layers:
        while used >= balance[stage]:
            stage, used = stage + 1, 0
        used += 1
        key = id(layer)
        if key not in first:
            first[key] = Location(stage, per_stage_count[stage])
            per_stage_count[stage] += 1
        locations.append(first[key])
    n = len(locations)
    invocations = [
        Invocation(k, locations[k], locations[k - 1] if k > 0 else None, locations[k + 1] if k + 1 < n else None) for k in range(n)
    ]
    return locations, invocations


class AsyncPipe(nn.Module):
    """Args:
        module: ``nn.Sequential`` (every rank builds everything and keeps its slice) or a list of
            :class:`LazyModule` (every rank builds only its slice).
        balance: layers per stage; stage ``r`` runs on group rank ``r``; further ranks stay idle.
        group: pipeline process group (default: the pipeline group of ``initialize_model_parallel`` if
            initialised, else WORLD).
        chunks / checkpoint / deferred_batch_norm: as for :class:`Pipe`.
    """

    def __init__(self, module: Union[nn.Sequential, List[LazyModule]], balance: Iterable[int], *, group: Any = None,
                 worker_map: Optional[Any] = None, input_device: Optional[torch.device] = None, chunks: int = 1,
                 checkpoint: str = "except_last", deferred_batch_norm: bool = False) -> None:
        super().__init__()
        if chunks <= 0:
            raise ValueError("number of chunks must be positive integer")
        if checkpoint not in ["always", "except_last", "never"]:
            raise ValueError("checkpoint is not one of 'always', 'except_last', or 'never'")
        if group is None:
            from ..model_parallel import initialize as mpi

            group = mpi.get_pipeline_parallel_group() if mpi.model_parallel_is_initialized() else dist.group.WORLD
        self.group = group
        self.balance = list(balance)
        self.chunks = chunks
        self.checkpoint = checkpoint
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if len(self.balance) > self.world:
            raise IndexError(f"too few ranks to hold given partitions (ranks: {self.world}, partitions: {len(self.balance)})")
        check_balance(module, self.balance)
        self.final_stage = len(self.balance) - 1
        self.pipeline: Optional[AsyncPipeline] = None
        entries = list(module)
        if len({id(l) for l in entries}) < len(entries):
            # a layer object that appears more than once: event-loop schedule, data may revisit a stage
            self._init_event_loop(entries, input_device, deferred_batch_norm)
            _refuse_lazy_skippables(module, [] if self.partition is None else [layer for seq in self.partition for layer in seq])
            return
        if self.rank >= len(self.balance):
            logging.warning(f"AsyncPipe: rank {self.rank} has no partition and stays idle")
            self.partition: Optional[nn.Sequential] = None
        else:
            lo = sum(self.balance[: self.rank])
            layers = list(module)[lo : lo + self.balance[self.rank]] if isinstance(module, nn.Sequential) else module[lo : lo + self.balance[self.rank]]
            built = [l() if isinstance(l, LazyModule) else l for l in layers]
            _refuse_lazy_skippables(module, built)
            part = nn.Sequential(*built)
            if deferred_batch_norm:
                part = DeferredBatchNorm.convert_deferred_batch_norm(part, chunks)
            self.partition = part
        if input_device is None:
            input_device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
        self.input_device = input_device
        if self.partition is not None:
            self.partition.to(self.input_device)
        self.transport = get_transport(group, self.input_device)
        self._outputs: List[Tensor] = []

    def _init_event_loop(self, entries: List[Any], input_device: Optional[torch.device], deferred_batch_norm: bool) -> None:
        locations, invocations = plan_invocations(entries, self.balance)
        if input_device is None:
            input_device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl" else torch.device("cpu")
        self.input_device = input_device
        self.transport = get_transport(self.group, self.input_device)
        wrappers: dict = {}
        for entry, loc, inv in zip(entries, locations, invocations):
            if loc.stage != self.rank:
                continue
            if loc not in wrappers:
                layer = entry() if isinstance(entry, LazyModule) else entry
                part = nn.Sequential(layer)
                if deferred_batch_norm:
                    part = DeferredBatchNorm.convert_deferred_batch_norm(part, self.chunks)
                wrappers[loc] = ModuleWrapper(part.to(self.input_device), loc)
            wrappers[loc].invocations.append(inv)
        mine = [wrappers[k] for k in sorted(wrappers, key=lambda l: l.index)]
        self.partition = nn.Sequential(*[w.module for w in mine]) if mine else None  # registers the parameters
        self._head_stage = invocations[0].this.stage
        self._tail_stage = invocations[-1].this.stage
        self._stages_in_use = sorted({loc.stage for loc in locations})
        self.pipeline = AsyncPipeline(mine, self.group, self.rank, self.transport)
        self._outputs = []

    def instantiate_partition(self, module: Union[nn.Sequential, List[LazyModule]], balance: List[int], group: Any = None) -> List[ModuleWrapper]:
        """This rank's layers as :class:`ModuleWrapper` objects with their invocations (lazy entries are built only if
        they live here).  ``AsyncPipe`` calls the planner itself when it meets a shared layer; the method is public for
        code that wants the plan (parity: fairscale/nn/pipe/async_pipe.py:224-319)."""
        entries = list(module)
        locations, invocations = plan_invocations(entries, balance)
        rank = dist.get_rank(group if group is not None else self.group)
        wrappers: dict = {}
        for entry, loc, inv in zip(entries, locations, invocations):
            if loc.stage != rank:
                continue
            if loc not in wrappers:
                layer = entry() if isinstance(entry, LazyModule) else entry
                wrappers[loc] = ModuleWrapper(nn.Sequential(layer), loc)
            wrappers[loc].invocations.append(inv)
        return [wrappers[k] for k in sorted(wrappers, key=lambda l: l.index)]

    def create_pipeline(self) -> AsyncPipeline:
        """The event-loop driver over this rank's layers (built on demand for a model without shared layers)."""
        if self.pipeline is None:
            parts = []
            if self.partition is not None:
                lo = sum(self.balance[: self.rank])
                n_total = sum(self.balance)
                loc = Location(self.rank, 0)
                src = Location(self.rank - 1, 0) if self.rank > 0 else None
                dst = Location(self.rank + 1, 0) if lo + len(self.partition) < n_total else None
                parts = [ModuleWrapper(self.partition, loc, [Invocation(self.rank, loc, src, dst)])]
            return AsyncPipeline(parts, self.group, self.rank, self.transport)
        return self.pipeline

    def _forward_event_loop(self, input: Optional[TensorOrTensors]) -> Optional[TensorOrTensors]:
        assert self.pipeline is not None
        if self.partition is None:
            return None
        if self.rank == self._head_stage:
            assert isinstance(input, Tensor), "the event-loop schedule moves single tensors"
            batches = [b.tensor for b in microbatch.scatter(input, self.chunks)]
            n = len(batches)
            for r in self._stages_in_use:
                if r != self.rank:
                    self.transport.send(torch.tensor([n], dtype=torch.int64, device=self.input_device), r)
        else:
            batches = None
            n = int(self.transport.recv(self._head_stage).item())
        self.pipeline.checkpoint_stop = {"always": n, "except_last": n - 1, "never": 0}[self.checkpoint]
        outs = self.pipeline.run(self.training, batches, n)
        if self.rank == self._tail_stage:
            assert outs is not None
            return torch.cat(outs)
        return None

    def __len__(self) -> int:
        return 0 if self.partition is None else len(self.partition)

    def _run_stage(self, x: TensorOrTensors, use_checkpoint: bool) -> TensorOrTensors:
        assert self.partition is not None
        if use_checkpoint and torch.is_grad_enabled():
            from .checkpoint import recomputed_in_backward

            return recomputed_in_backward(self.partition, x)
        return self.partition(x)

    def forward(self, input: Optional[TensorOrTensors] = None) -> Optional[TensorOrTensors]:  # type: ignore[override]
        """Stage 0 consumes ``input``; the final stage returns the gathered output; other stages return the list
        of their micro-batch outputs (pass it to :meth:`back_helper` to run their share of backward)."""
        if self.pipeline is not None:
            return self._forward_event_loop(input)
        if self.partition is None:
            return None
        first, last = self.rank == 0, self.rank == self.final_stage
        if first:
            assert input is not None
            microbatch.check(input)
            batches = [b.tensor_or_tensors for b in microbatch.scatter(input, self.chunks)]
            n = len(batches)
            if not last:
                self.transport.send(torch.tensor([n], dtype=torch.int64, device=self.input_device), self.rank + 1)
        else:
            n = int(self.transport.recv(self.rank - 1).item())
            if not last:
                self.transport.send(torch.tensor([n], dtype=torch.int64, device=self.input_device), self.rank + 1)
        stop = {"always": n, "except_last": n - 1, "never": 0}[self.checkpoint] if self.training else 0
        outs: List[Tensor] = []
        for i in range(n):
            if first:
                x = batches[i]
            else:
                x = self.transport.recv(self.rank - 1, slot=i)
                if i + 1 < n:
                    self.transport.prefetch(self.rank - 1, i + 1)  # the next activation travels while this one is computed on
                if x.requires_grad and torch.is_grad_enabled():
                    x = _RecvBoundary.apply(x, self.transport, self.rank - 1, n + i)  # gradient slots follow the activation slots
            y = self._run_stage(x, i < stop)
            assert isinstance(y, Tensor), "stages of AsyncPipe exchange single tensors"
            if not last:
                self.transport.send(y, self.rank + 1, slot=i)
            outs.append(y)
        self._outputs = outs
        if last:
            return torch.cat(outs)
        return outs  # type: ignore[return-value]

    def back_helper(self, output: Optional[List[Tensor]] = None) -> None:
        """Run backward on a non-final stage: receive each micro-batch's output gradient from the next stage
        (reverse order) and back-propagate; gradients for the previous stage leave through the recv boundary."""
        if self.pipeline is not None:
            # event-loop schedule: every rank (the last one too, after its loss.backward()) collects the gradients of
            # the activations it sent away
            self.pipeline.back()
            return
        if self.partition is None or self.rank == self.final_stage:
            self.transport.flush()
            return
        outs = self._outputs if output is None else output
        n = len(outs)
        # the next stage emits the gradients in its backward order (the final stage back-propagates torch.cat(outs), i.e. in
        # autograd's reverse order): last micro-batch first.  The receive of the following gradient is posted before the
        # backward of the current one.
        slots = [n + (n - 1 - k) for k in range(n)]
        for k, y in enumerate(reversed(outs)):
            g = self.transport.recv(self.rank + 1, slot=slots[k])
            if k + 1 < n:
                self.transport.prefetch(self.rank + 1, slots[k + 1])
            if y.requires_grad:
                torch.autograd.backward(y, g)
        self.transport.flush()
