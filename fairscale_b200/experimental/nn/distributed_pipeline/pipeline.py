"""Driver of the RPC pipeline (parity: fairscale/experimental/nn/distributed_pipeline/pipeline.py:33-202)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Union

import torch
from torch import Tensor, nn
from torch.distributed import rpc

from ....nn.pipe import microbatch
from .data import DataConsumer
from .graph import Node, PipelineModulesGraph
from .partition_handler import PartitionHandler, feed_record_async

Device = Union[torch.device, int, str]
MOVING_DENIED = TypeError("denied to move parameters and buffers, because DistributedPipeline should manage device placement")


def check_pytorch_version() -> None:
    from ....internal.version import torch_version

    if torch_version() < (1, 8, 0):
        raise Exception("DistributedPipeline requires PyTorch version 1.8 or higher")


class DistributedPipeline(nn.Module):
    """GPipe-style synchronous pipeline over modules that live on RPC workers.

    Args: ``graph`` (:class:`PipelineModulesGraph`), ``chunks`` micro-batches per mini-batch, ``checkpoint`` in
    ``'always' | 'except_last' | 'never'``.  ``forward`` returns an RRef to the output on the last partition's
    worker; train with ``torch.distributed.autograd`` and ``DistributedOptimizer(parameter_rrefs())``.

    Every worker process should import this package before ``rpc.init_rpc``: an RPC agent unpickles incoming calls on
    several threads, and letting those threads perform the first import concurrently can fail inside the import lock.
    """

    DataConsumer = DataConsumer  # the edge record type, reachable from the class as in the reference

    @dataclass
    class Partition:
        nodes: List[Node]
        handler: rpc.RRef

        def __hash__(self) -> int:
            return id(self)

    def __init__(self, graph: PipelineModulesGraph, chunks: int = 1, checkpoint: str = "except_last") -> None:
        super().__init__()
        chunks = int(chunks)
        if chunks <= 0:
            raise ValueError("number of chunks must be positive integer")
        if checkpoint not in ["always", "except_last", "never"]:
            raise ValueError("checkpoint is not one of 'always', 'except_last', or 'never'")
        self.chunks = chunks
        stop = {"always": chunks, "except_last": chunks - 1, "never": 0}[checkpoint]
        self.partitions = [
            self.Partition(nodes, rpc.remote(mod.owner(), PartitionHandler, args=(
                mod, nodes[0].module.device, len(nodes[0].inputs), nodes[-1].num_outputs, i, chunks, stop)))
            for i, (nodes, mod) in enumerate(graph.partition_graph())
        ]
        self.input_consumers = [
            DataConsumer(next(p for p in self.partitions if p.nodes[0] is c.consumer), c.consumer_input_idx, c.output_idx)
            for c in graph.model_input_consumers
        ]
        self.graph = graph

    def cuda(self, device: Optional[Device] = None) -> "DistributedPipeline":
        raise MOVING_DENIED

    def cpu(self) -> "DistributedPipeline":
        raise MOVING_DENIED

    def to(self, *args: Any, **kwargs: Any) -> "DistributedPipeline":
        if "device" in kwargs or "tensor" in kwargs or (args and (isinstance(args[0], (torch.device, int, str)) or torch.is_tensor(args[0]))):
            raise MOVING_DENIED
        return super().to(*args, **kwargs)

    def parameter_rrefs(self) -> List[rpc.RRef]:
        out: List[rpc.RRef] = []
        for p in self.partitions:
            out.extend(p.handler.rpc_sync().local_parameter_rrefs())
        return out

    def forward(self, *inputs: Tensor) -> rpc.RRef:  # type: ignore[override]
        for x in inputs:
            microbatch.check(x)
        batches = [microbatch.scatter(x, self.chunks) for x in inputs]
        records: Dict[DistributedPipeline.Partition, rpc.RRef] = {}
        result = None
        for part in reversed(self.partitions):  # consumers' records must exist before their producers start
            h = part.handler.remote()
            consumers = []
            for c in part.nodes[-1].output_consumers:
                cp = next(p for p in self.partitions if p.nodes[0] is c.consumer)
                consumers.append(DataConsumer(records[cp], c.consumer_input_idx, c.output_idx))
            records[part] = h.make_pipeline_record(consumers, len(batches[0]))
            r = h.run_pipeline(records[part])
            if part is self.partitions[-1]:
                result = r
        futs = []
        for i, mb in enumerate(zip(*batches)):
            for ic in self.input_consumers:
                futs.append(feed_record_async(records[ic.consumer], i, ic.consumer_input_idx, mb[ic.output_idx].tensor))
        for f in futs:
            f.wait()
        assert result is not None
        return result
