"""Split an arbitrary model into a sequence of ``torch.fx.GraphModule`` shards of similar parameter count.

Capability parity with fairscale/experimental/nn/auto_shard.py:43-225 (``shard_model(model, shard_count)``,
automatic leaf-wrapping of sub-modules fx cannot trace; the result feeds ``OffloadModel`` or a pipeline).

The cut points are found differently: the traced graph is scanned once to compute, for every position, the set of
values that are still needed later (liveness).  A position is a legal cut only when exactly one value crosses it,
so a cut never lands inside a residual branch, and no repair pass that merges shards backwards is needed.  Among
the legal cuts, the ones closest to the ideal cumulative parameter counts ``k * total / shard_count`` are taken.
"""

from __future__ import annotations

import logging
from typing import Dict, List, Set

import torch
import torch.fx
from torch.fx.node import Node


class _ExtendedLeafTracer(torch.fx.Tracer):
    """Tracer that also treats the given module instances as leaves."""

    def __init__(self, leaf_modules: Set[torch.nn.Module]):
        super().__init__()
        self.leaf_modules = leaf_modules

    def is_leaf_module(self, m: torch.nn.Module, model_qualified_name: str) -> bool:
        return super().is_leaf_module(m, model_qualified_name) or m in self.leaf_modules


def _trace(model: torch.nn.Module) -> torch.fx.GraphModule:
    """Trace ``model``; any sub-module that cannot be traced symbolically becomes a leaf call."""
    leaves: Set[torch.nn.Module] = set()
    tracer = _ExtendedLeafTracer(leaves)
    for _, module in model.named_modules():
        if module is model or tracer.is_leaf_module(module, ""):
            continue
        try:
            _ExtendedLeafTracer(leaves).trace(module)
        except Exception:  # fx raises TypeError / TraceError / others on data-dependent control flow
            leaves.add(module)
    tracer = _ExtendedLeafTracer(leaves)
    return torch.fx.GraphModule(model, tracer.trace(model))


def _node_params(gm: torch.fx.GraphModule, node: Node, seen: Set[int]) -> int:
    """Parameters first touched by ``node`` (a shared parameter counts where it is used first)."""
    tensors = []
    if node.op == "call_module":
        tensors = list(gm.get_submodule(node.target).parameters())  # type: ignore[arg-type]
    elif node.op == "get_attr":
        obj = gm
        for part in str(node.target).split("."):
            obj = getattr(obj, part)
        if isinstance(obj, torch.nn.Parameter):
            tensors = [obj]
    n = 0
    for t in tensors:
        if id(t) not in seen:
            seen.add(id(t))
            n += t.numel()
    return n


def _legal_cuts(nodes: List[Node]) -> List[int]:
    """Indices ``i`` such that cutting after ``nodes[i]`` hands exactly one value (``nodes[i]``) to the rest."""
    last_use: Dict[Node, int] = {}
    for i, n in enumerate(nodes):
        for a in n.all_input_nodes:
            last_use[a] = i
    legal = []
    live: Set[Node] = set()
    for i, n in enumerate(nodes[:-1]):
        live.add(n)
        live = {v for v in live if last_use.get(v, -1) > i}
        if live == {n} and n.op != "placeholder":
            legal.append(i)
    return legal


def shard_model(model: torch.nn.Module, shard_count: int = 3) -> List[torch.fx.GraphModule]:
    """Return up to ``shard_count`` GraphModules whose composition equals ``model``.

    Every shard but the first takes one input: the single output of the previous shard.  Fewer shards are returned
    when the model has fewer legal cut points (e.g. long-range skip connections)."""
    gm = _trace(model)
    nodes = [n for n in gm.graph.nodes]
    body = [n for n in nodes if n.op != "output"]
    seen: Set[int] = set()
    cum, total = [], 0
    for n in body:
        total += _node_params(gm, n, seen)
        cum.append(total)
    logging.info(f"Total number of params are {total}")
    legal = _legal_cuts(body)
    cuts: List[int] = []
    for k in range(1, shard_count):
        want = k * total / shard_count
        cands = [i for i in legal if (not cuts or i > cuts[-1])]
        if not cands:
            break
        best = min(cands, key=lambda i: (abs(cum[i] - want), i))
        # a cut that adds no parameters to the shard before it is pointless
        if cum[best] > (cum[cuts[-1]] if cuts else 0) and cum[best] < total:
            cuts.append(best)
    shards: List[torch.fx.GraphModule] = []
    start = 0
    bounds = cuts + [len(body) - 1]
    prev_out: Node = None  # type: ignore[assignment]
    for si, end in enumerate(bounds):
        g = torch.fx.Graph()
        env: Dict[Node, Node] = {}
        if si > 0:
            env[prev_out] = g.placeholder(f"shard_input_{si}")
        for n in body[start : end + 1]:
            if n.op == "placeholder" and si > 0:
                raise RuntimeError("model inputs must all be consumed by the first shard")
            env[n] = g.node_copy(n, lambda x: env[x])
        if si == len(bounds) - 1:
            out_node = nodes[-1]
            g.output(torch.fx.node.map_arg(out_node.args[0], lambda x: env[x]))
        else:
            g.output(env[body[end]])
        shards.append(torch.fx.GraphModule(gm, g))
        prev_out = body[end]
        start = end + 1
    return shards
