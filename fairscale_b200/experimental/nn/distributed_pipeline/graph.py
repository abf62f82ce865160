"""Data-flow graph of remote modules and its split into pipeline partitions.

Parity: fairscale/experimental/nn/distributed_pipeline/graph.py:17-207 (``add_layer``, ``add_sequence``,
``partition_graph``: maximal chains of single-input / single-output modules on one worker and device become one
partition).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Set, Tuple, Union

from torch import Tensor, nn
from torch.distributed import rpc

from .data import DataConsumer


class MultiInputSequential(nn.Module):
    """``nn.Sequential`` whose first module may take several inputs."""

    def __init__(self, *modules: nn.Module) -> None:
        super().__init__()
        self.modules_list = nn.ModuleList(modules)

    def forward(self, *inputs: Tensor) -> Any:  # type: ignore[override]
        x = self.modules_list[0](*inputs)
        for m in self.modules_list[1:]:
            x = m(x)
        return x


def RemoteSequential(rref_list: List[rpc.RRef]) -> MultiInputSequential:
    return MultiInputSequential(*(r.local_value() for r in rref_list))


@dataclass
class DataSource:
    producer: Optional["Node"]  # None: an input of the whole model
    output_idx: int


class Node:
    def __init__(self, module: Any):
        self.module = module
        self.num_outputs: Optional[int] = None
        self.inputs: List[DataSource] = []
        self.output_consumers: List[DataConsumer["Node"]] = []


DataSourceSpec = Union[int, Any, Tuple[Any, int]]


class PipelineModulesGraph(nn.Module):
    """Remote modules plus which model input / module output feeds which module input."""

    DataSourceSpec = DataSourceSpec

    def __init__(self) -> None:
        super().__init__()
        self.nodes: List[Node] = []

    def _find_node(self, module: Any) -> Node:
        for n in self.nodes:
            if n.module is module:
                return n
        raise ValueError("module was not added to the graph")

    def _source(self, spec: DataSourceSpec) -> DataSource:
        if isinstance(spec, int):
            return DataSource(None, spec)
        if isinstance(spec, tuple):
            return DataSource(self._find_node(spec[0]), spec[1])
        return DataSource(self._find_node(spec), 0)

    def add_layer(self, module: Any, inputs: List[DataSourceSpec], num_outputs: Optional[int] = None) -> None:
        """Add ``module``; each input is a model-input index, an earlier module, or ``(earlier module, output index)``.
        ``num_outputs`` is the tuple length when the module returns a tuple."""
        node = Node(module)
        node.inputs = [self._source(s) for s in inputs]
        node.num_outputs = num_outputs
        self.nodes.append(node)

    def add_sequence(self, modules: List[Any], first_module_inputs: List[DataSourceSpec], last_module_num_outputs: Optional[int] = None) -> None:
        """Add a chain: every module feeds the next one."""
        nxt = first_module_inputs
        for i, m in enumerate(modules):
            self.add_layer(m, nxt, last_module_num_outputs if i == len(modules) - 1 else None)
            nxt = [m]

    def _compile(self) -> None:
        self.model_input_consumers: List[DataConsumer[Node]] = []
        for node in self.nodes:
            node.output_consumers = []
        for node in self.nodes:
            for idx, src in enumerate(node.inputs):
                c = DataConsumer(node, idx, src.output_idx)
                (src.producer.output_consumers if src.producer is not None else self.model_input_consumers).append(c)

    def _chain_from(self, node: Node) -> List[Node]:
        chain, cur = [], node
        while True:
            chain.append(cur)
            if len(cur.output_consumers) != 1 or cur.num_outputs is not None:
                break
            nxt = cur.output_consumers[0].consumer
            if nxt.inputs != [DataSource(cur, 0)] or nxt.module.on != cur.module.on or nxt.module.device != cur.module.device:
                break
            cur = nxt
        return chain

    def partition_graph(self) -> List[Tuple[List[Node], rpc.RRef]]:
        """[(nodes of the partition, RRef to the nn.Module that runs them on their owner)]."""
        self._compile()
        used: Set[int] = set()
        parts = []
        for node in self.nodes:
            if id(node) in used:
                continue
            chain = self._chain_from(node)
            assert not used.intersection(id(n) for n in chain)
            used.update(id(n) for n in chain)
            if len(chain) == 1:
                mod = chain[0].module.get_module_rref()
            else:
                mod = rpc.remote(chain[0].module.on, RemoteSequential, args=([n.module.get_module_rref() for n in chain],))
            parts.append((chain, mod))
        return parts
