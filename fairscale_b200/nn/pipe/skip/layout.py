"""Static routing table of skip tensors across partitions (parity: fairscale/nn/pipe/skip/layout.py:30-125)."""

from __future__ import annotations

from typing import Dict, Iterable, List, Tuple

from torch import nn

from .namespace import Namespace

__all__: List[str] = []


class SkipLayout:
    """For every skip tensor: the partition that stashes it and the partition that pops it."""

    def __init__(self, num_partitions: int, skip_routes: Dict[Tuple[Namespace, str], Tuple[int, int]]) -> None:
        self.by_ns_name = skip_routes
        # by_partition[j] lists (prev_j, ns, name) of the tensors popped in partition j, sorted for determinism
        self.by_partition: List[List[Tuple[int, Namespace, str]]] = [[] for _ in range(num_partitions)]
        for (ns, name), (prev_j, next_j) in skip_routes.items():
            self.by_partition[next_j].append((prev_j, ns, name))
        for entries in self.by_partition:
            entries.sort()

    def copy_policy(self, next_j: int) -> Iterable[Tuple[int, Namespace, str]]:
        """Skip tensors that must be copied into partition ``next_j`` from an earlier partition."""
        for prev_j, ns, name in self.by_partition[next_j]:
            if prev_j != next_j:
                yield prev_j, ns, name

    def copy_policy_by_src(self, prev_j: int) -> Iterable[Tuple[int, Namespace, str]]:
        """Skip tensors stashed in partition ``prev_j`` that must be copied to a later partition: ``(next_j, ns, name)``,
        sorted by destination."""
        out = [(next_j, ns, name) for (ns, name), (src, next_j) in self.by_ns_name.items() if src == prev_j and next_j != prev_j]
        out.sort(key=lambda e: (e[0], e[2]))
        return iter(out)

    def requires_copy(self, ns: Namespace, name: str) -> bool:
        """False when stash and pop happen in the same partition (or the tensor is unknown)."""
        prev_j, next_j = self.by_ns_name.get((ns, name), (-1, -1))
        return prev_j != next_j


def inspect_skip_layout(partitions: List[nn.Sequential]) -> SkipLayout:
    """Scan the partitions for skippable layers and record where each skip tensor is stashed and popped."""
    from .skippable import Skippable

    routes: Dict[Tuple[Namespace, str], Tuple[int, int]] = {}
    stashed_at: Dict[Tuple[Namespace, str], int] = {}
    for j, partition in enumerate(partitions):
        for layer in partition:
            if not isinstance(layer, Skippable):
                continue
            for ns, name in layer.stashable():
                stashed_at[(ns, name)] = j
            for ns, name in layer.poppable():
                routes[(ns, name)] = (stashed_at.pop((ns, name)), j)
    return SkipLayout(len(partitions), routes)
