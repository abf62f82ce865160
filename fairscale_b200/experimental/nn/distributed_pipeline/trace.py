"""Build a :class:`PipelineModulesGraph` from a model made of ``RemoteModule`` calls with ``torch.fx``.

Parity: fairscale/experimental/nn/distributed_pipeline/trace.py:12-107.  Only calls of remote modules, tuple
indexing of their results and model inputs may appear in ``forward``.
"""

from __future__ import annotations

import inspect
import operator
from typing import Any, Dict, List, Optional, Tuple

import torch.fx
import torch.nn as nn
from torch.distributed.nn import RemoteModule

from .graph import PipelineModulesGraph


class RemoteModuleTracer(torch.fx.Tracer):
    def is_leaf_module(self, m: nn.Module, module_qualified_name: str) -> bool:
        return isinstance(m, RemoteModule)


def make_graph(module: nn.Module) -> PipelineModulesGraph:
    tracer = RemoteModuleTracer()
    saved = (RemoteModule.named_modules, RemoteModule.named_children)
    try:  # RemoteModule refuses to enumerate children; the tracer only needs the plain nn.Module behaviour
        RemoteModule.named_modules = nn.Module.named_modules  # type: ignore[method-assign]
        RemoteModule.named_children = nn.Module.named_children  # type: ignore[method-assign]
        fx_graph = tracer.trace(module)
    finally:
        RemoteModule.named_modules, RemoteModule.named_children = saved  # type: ignore[method-assign]
    arg_names = list(inspect.signature(module.forward).parameters)
    data: Dict[torch.fx.Node, Any] = {}
    calls: List[Tuple[torch.fx.Node, RemoteModule]] = []
    for node in fx_graph.nodes:
        if node.op == "call_module":
            m: Any = module
            for part in str(node.target).split("."):
                m = getattr(m, part)
            assert isinstance(m, RemoteModule), f"{node.target} is not a RemoteModule"
            data[node] = m
            calls.append((node, m))
        elif node.op == "call_function" and node.target == operator.getitem:
            src = data[node.args[0]]
            assert isinstance(src, RemoteModule)
            data[node] = (src, node.args[1])
        elif node.op == "placeholder":
            data[node] = arg_names.index(node.target)
        elif node.op != "output":
            raise AssertionError(f"Invalid node {node}: every tensor operation must be done by a RemoteModule")
    num_outputs: Dict[Any, Optional[int]] = {}
    for node, _ in calls:
        for arg in node.args:
            d = data[arg]
            if isinstance(d, tuple):
                num_outputs[d[0]] = max(num_outputs.get(d[0]) or 0, d[1] + 1)
            elif not isinstance(d, int):
                assert num_outputs.get(d) is None
                num_outputs[d] = None
    graph = PipelineModulesGraph()
    for node, m in calls:
        graph.add_layer(m, [data[a] for a in node.args], num_outputs.get(m))
    return graph
