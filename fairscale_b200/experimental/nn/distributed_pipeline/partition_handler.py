"""Worker-side execution of one pipeline partition.

Parity: fairscale/experimental/nn/distributed_pipeline/partition_handler.py:27-291.  A record holds the inputs of
one mini-batch (fed chunk by chunk from upstream partitions or from the driver); ``run_pipeline`` processes the
chunks in order on the RPC thread that called it and feeds downstream records as soon as a chunk is done, so
consecutive partitions work on different chunks at the same time.
"""

from __future__ import annotations

from threading import Condition
from typing import Any, Dict, List, Optional

import torch
from torch import Tensor
from torch.autograd.profiler import record_function
from torch.distributed import rpc

from .data import DataConsumer


class DistributedPipelineRecord:
    def __init__(self, device: torch.device, rank: int, chunks: int, num_inputs: int, num_outputs: Optional[int],
                 consumers: List[DataConsumer]) -> None:
        self.ready_cv = Condition()
        self.tensors: List[List[Optional[Tensor]]] = [[None] * num_inputs for _ in range(chunks)]
        self.recv_events: List[List[Any]] = [[None] * num_inputs for _ in range(chunks)]
        self.outputs: List[Any] = [None] * chunks
        self.chunks = chunks  # micro-batches of THIS mini-batch: fewer than the pipeline's setting when the batch is small
        self.consumers = consumers
        self.rank = rank
        self.device = device
        self.pending: List[Any] = []

    def __getstate__(self) -> Dict:
        return {}

    def feed(self, chunk: int, input_idx: int, input: Tensor) -> None:
        """Called (remotely) by the producer of input ``input_idx`` of micro-batch ``chunk``."""
        if input.device != self.device:
            input = input.to(self.device, non_blocking=True)
        ev = torch.cuda.current_stream(input.device).record_event() if input.is_cuda else None
        with self.ready_cv:
            assert self.tensors[chunk][input_idx] is None, "input fed twice"
            self.tensors[chunk][input_idx] = input
            self.recv_events[chunk][input_idx] = ev
            self.ready_cv.notify_all()

    def wait_for(self, chunk: int) -> List[Tensor]:
        with self.ready_cv:
            while any(t is None for t in self.tensors[chunk]):
                self.ready_cv.wait()
        for ev in self.recv_events[chunk]:
            if ev is not None:
                torch.cuda.current_stream(self.device).wait_event(ev)
        return self.tensors[chunk]  # type: ignore[return-value]

    def forward_results(self, chunk: int) -> None:
        out = self.outputs[chunk]
        for c in self.consumers:
            if c.consumer.is_owner():
                # the next partition lives in this process: hand the tensor over directly (no copy, no RPC to oneself, and
                # the autograd graph of the two partitions stays one local graph)
                c.consumer.local_value().feed(chunk, c.consumer_input_idx, out[c.output_idx])
            else:
                self.pending.append(feed_record_async(c.consumer, chunk, c.consumer_input_idx, out[c.output_idx]))


def _feed_record(record_rref: rpc.RRef, chunk: int, input_idx: int, tensor: Tensor) -> None:
    record_rref.local_value().feed(chunk, input_idx, tensor)


def feed_record_async(record_rref: rpc.RRef, chunk: int, input_idx: int, tensor: Tensor) -> Any:
    """Send ``tensor`` to the record behind ``record_rref``; returns the future of the call.

    The call is issued with ``rpc.rpc_async`` from the calling thread.  ``record_rref.rpc_async().feed(...)`` would not do: the
    RRef proxy first fetches the type of the remote object and issues the real call from the callback of that fetch, on a
    thread that does not carry the caller's distributed-autograd context - the first tensors of a mini-batch then travel
    without their autograd edge, arrive as leaves, and the backward pass waits for gradients that never come."""
    return rpc.rpc_async(record_rref.owner(), _feed_record, args=(record_rref, chunk, input_idx, tensor))


class PartitionHandler:
    def __init__(self, module_rref: rpc.RRef, device: str, num_inputs: int, num_outputs: Optional[int], rank: int,
                 chunks: int, checkpoint_stop: int) -> None:
        self.module = module_rref.local_value()
        self.chunks = chunks
        self.device = torch.device(device)
        self.checkpoint_stop = checkpoint_stop
        self.rank = rank
        self.num_inputs = num_inputs
        self.num_outputs = num_outputs

    def __getstate__(self) -> Dict:
        return {}

    def local_parameter_rrefs(self) -> List[rpc.RRef]:
        return [rpc.RRef(p) for p in self.module.parameters()]

    def make_pipeline_record(self, consumers: List[DataConsumer], chunks: Optional[int] = None) -> DistributedPipelineRecord:
        """``chunks``: how many micro-batches the driver will feed (a mini-batch with fewer rows than the configured number of
        chunks gives fewer; waiting for the configured number would never end)."""
        n = self.chunks if chunks is None else min(int(chunks), self.chunks)
        return DistributedPipelineRecord(self.device, self.rank, n, self.num_inputs, self.num_outputs, consumers)

    def _compute(self, inputs: List[Tensor], chunk: int, chunks: Optional[int] = None) -> Any:
        def fn(*xs: Tensor) -> Any:
            with record_function("chunk%d-rank%d" % (chunk, self.rank)):
                y = self.module(*xs)
            return tuple(y) if self.num_outputs is not None else (y,)

        # "except_last" leaves the last micro-batch of this mini-batch alone, however many there are
        missing = self.chunks - (self.chunks if chunks is None else chunks)
        stop = max(0, self.checkpoint_stop - missing) if self.module.training else 0
        if chunk < stop and torch.is_grad_enabled() and any(x.requires_grad for x in inputs):
            from torch.utils.checkpoint import checkpoint

            return checkpoint(fn, *inputs, use_reentrant=False)
        return fn(*inputs)

    def run_pipeline(self, pipeline_record_rref: rpc.RRef) -> Optional[Tensor]:
        """Process every chunk of the mini-batch; the last partition returns the concatenated model output."""
        rec: DistributedPipelineRecord = pipeline_record_rref.local_value()
        for chunk in range(rec.chunks):
            with record_function("feed"):
                inputs = rec.wait_for(chunk)
            rec.outputs[chunk] = self._compute(inputs, chunk, rec.chunks)
            rec.forward_results(chunk)
        for f in rec.pending:
            f.wait()
        result = None
        if not rec.consumers:
            outs = [o for o in rec.outputs if o is not None]
            assert all(len(o) == 1 for o in outs)
            result = torch.cat([o[0] for o in outs])
            if result.is_cuda:
                torch.cuda.current_stream(result.device).synchronize()
        rec.outputs = []
        return result
