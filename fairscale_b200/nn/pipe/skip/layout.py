"""Where every skip tensor of a partitioned model is produced and consumed.

Skip tensors that stay inside one partition never leave the module code.  A skip tensor that is stashed in partition
``a`` and popped in partition ``b > a`` is a *route*: the pipeline treats it as an extra output port of stage ``a`` and
an extra input port of stage ``b`` (so checkpointing, copies between devices and autograd handle it like any other
activation) and moves it straight from device ``a`` to device ``b``.  ``SkipLayout`` answers the questions the pipeline
asks about routes; same query interface as fairscale/nn/pipe/skip/layout.py:17-92.
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Tuple

from torch import nn

from .namespace import Namespace

__all__: List[str] = []

SkipKey = Tuple[Optional[Namespace], str]


def _order(key: SkipKey) -> Tuple[int, str]:
    ns, name = key
    return (-1 if ns is None else ns.id, name)


class SkipLayout:
    def __init__(self, num_partitions: int, skip_routes: Dict[SkipKey, Tuple[int, int]]) -> None:
        self.num_partitions = num_partitions
        self.skip_routes = skip_routes  # (namespace, name) -> (stashing partition, popping partition)
        self._imports: List[List[SkipKey]] = [[] for _ in range(num_partitions)]
        self._exports: List[List[SkipKey]] = [[] for _ in range(num_partitions)]
        for key in sorted(skip_routes, key=_order):
            src, dst = skip_routes[key]
            if src != dst:
                self._exports[src].append(key)
                self._imports[dst].append(key)

    def imports(self, partition: int) -> List[SkipKey]:
        """Skip tensors that arrive at ``partition`` from earlier partitions, in port order."""
        return self._imports[partition]

    def exports(self, partition: int) -> List[SkipKey]:
        """Skip tensors that ``partition`` stashes for later partitions, in port order."""
        return self._exports[partition]

    def copy_policy(self, next_j: int) -> Iterable[Tuple[int, Optional[Namespace], str]]:
        """``(source partition, namespace, name)`` of every skip tensor that has to be brought to partition ``next_j``."""
        for ns, name in self._imports[next_j]:
            yield (self.skip_routes[(ns, name)][0], ns, name)

    def copy_policy_by_src(self, prev_j: int) -> Iterable[Tuple[int, Optional[Namespace], str]]:
        """``(destination partition, namespace, name)`` of every skip tensor that leaves partition ``prev_j``."""
        for ns, name in self._exports[prev_j]:
            yield (self.skip_routes[(ns, name)][1], ns, name)

    def requires_copy(self, ns: Optional[Namespace], name: str) -> bool:
        """Whether the skip tensor crosses a partition boundary."""
        src, dst = self.skip_routes.get((ns, name), (-1, -1))
        return src != dst


def inspect_skip_layout(partitions: List[nn.Sequential]) -> SkipLayout:
    """Walk the partitions in order and pair every stash with the pop that consumes it."""
    from .skippable import Skippable

    stashed_in: Dict[SkipKey, int] = {}
    routes: Dict[SkipKey, Tuple[int, int]] = {}
    for j, partition in enumerate(partitions):
        for layer in partition:
            if not isinstance(layer, Skippable):
                continue
            for key in layer.stashable():
                stashed_in[key] = j
            for key in layer.poppable():
                routes[key] = (stashed_in.pop(key), j)
    return SkipLayout(len(partitions), routes)
