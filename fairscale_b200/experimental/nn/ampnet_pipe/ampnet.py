"""Asynchronous pipeline event loop: no bubble, stale weights, optimizer steps inside the loop.

Capability parity with fairscale/experimental/nn/ampnet_pipe/ampnet.py:76-377 (AMPnet, arXiv:1705.09786): every
stage runs one forward and one backward per iteration once the pipeline is full (stage ``s`` of ``N`` first runs
``N - 1 - s`` forwards), applies its optimizer every ``min_update_interval`` gradients without waiting for the
other stages, and with ``weight_prediction`` lets the optimizer extrapolate the weights before each pass through
``optimizer.update_weight_using_future_predictions(rank, N, index, chunks, forward=...)``.

One loop serves head, trunk and tail stages (the reference has three copies); activations and gradients travel
through the asynchronous-send transport of ``AsyncPipe``.
"""

from __future__ import annotations

from typing import Any, Dict, Iterator, Tuple

import torch
from torch import nn
from torch.autograd.profiler import record_function

from ....nn.pipe.messages import SendRecvTransport


class AsyncAMPnetEventLoop:
    def __init__(self, partition: nn.Module, rank: int, n_stages: int, transport: SendRecvTransport, min_update_interval: int,
                 weight_prediction: bool, checkpoint_stop: int, input_device: Any, chunks: int):
        self.partition = partition
        self.rank, self.n = rank, n_stages
        self.transport = transport
        self.min_update_interval = min_update_interval
        self.weight_prediction = weight_prediction
        self.checkpoint_stop = checkpoint_stop
        self.input_device = input_device
        self.chunks = chunks

    def perform_optimizer_step(self, optimizer: Any, num_gradients: int) -> bool:
        if optimizer is None:
            return False
        if self.weight_prediction:
            return num_gradients % self.chunks == 0
        return num_gradients % self.min_update_interval == 0

    # ------------------------------------------------------------------ one forward / one backward
    def _forward(self, x: torch.Tensor, index: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Run the stage on micro-batch ``index``; returns (leaf input, output)."""
        leaf = x.detach()
        if leaf.is_floating_point() and self.rank > 0:
            leaf.requires_grad_()
        with record_function("chunk%d-part%d" % (index, self.rank)):
            if index < self.checkpoint_stop:
                from torch.utils.checkpoint import checkpoint

                out = checkpoint(self.partition, leaf, use_reentrant=False)
            else:
                out = self.partition(leaf)
        return leaf, out

    def _maybe_predict(self, optimizer: Any, index: int, forward: bool) -> None:
        if self.weight_prediction:
            optimizer.update_weight_using_future_predictions(self.rank, self.n, index, self.chunks, forward=forward)

    def _maybe_step(self, optimizer: Any, num_gradients: int, delegate: Any) -> None:
        if self.perform_optimizer_step(optimizer, num_gradients):
            optimizer.step()
            optimizer.zero_grad()
            delegate.check_and_save_weights(num_gradients)

    # ------------------------------------------------------------------ the loop
    def run(self, dataloader: Any, criterion: nn.Module, optimizer: Any, delegate: Any) -> None:
        """One epoch on this stage.  ``delegate`` provides ``transform_input``, ``transform_target``,
        ``transform_output_before_loss``, ``log_loss`` and ``check_and_save_weights``."""
        first, last = self.rank == 0, self.rank == self.n - 1
        it: Iterator[Any] = iter(dataloader)
        pending: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        sent = done = 0
        exhausted = False
        warmup = self.n - 1 - self.rank

        def forward_one() -> bool:
            nonlocal sent, exhausted
            try:
                batch = next(it)
            except StopIteration:
                exhausted = True
                return False
            self._maybe_predict(optimizer, sent, True)
            if first:
                x = delegate.transform_input(batch).to(self.input_device)
            else:
                x = self.transport.recv(self.rank - 1)
            leaf, out = self._forward(x, sent)
            if last:
                target = delegate.transform_target(batch).to(self.input_device)
                loss = criterion(delegate.transform_output_before_loss(out), target)
                pending[sent] = (leaf, loss)
                delegate.log_loss(batch, loss, sent)
            else:
                self.transport.send(out, self.rank + 1)
                pending[sent] = (leaf, out)
            sent += 1
            return True

        def backward_one() -> None:
            nonlocal done
            leaf, out = pending.pop(done)
            self._maybe_predict(optimizer, done, False)
            if last:
                out.backward()
            else:
                grad = self.transport.recv(self.rank + 1)
                if out.requires_grad:
                    out.backward(grad)
            if not first:
                g = leaf.grad if leaf.grad is not None else torch.zeros_like(leaf)
                self.transport.send(g, self.rank - 1)
            done += 1
            self._maybe_step(optimizer, done, delegate)

        # In-flight micro-batches were computed with weights the optimizer has since updated in place.  Under this
        # context autograd keeps a copy of a saved weight at the moment it is overwritten, so each backward uses
        # the weights of its own forward (weight stashing) whatever optimizer is used.
        with torch.autograd.graph.allow_mutation_on_saved_tensors():
            for _ in range(warmup):  # fill the pipeline
                if not forward_one():
                    break
            while not exhausted:  # steady state: one forward, one backward
                if forward_one():
                    backward_one()
            while pending:  # drain
                backward_one()
        self.transport.flush()
