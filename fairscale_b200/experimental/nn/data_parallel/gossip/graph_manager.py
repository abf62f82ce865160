"""Peer-to-peer communication topologies for gossip averaging.

Capability parity with fairscale/experimental/nn/data_parallel/gossip/graph_manager.py:17-289 (the same family of
graphs and the same rotation of out-peers).  An edge here is only a (src, dest) pair of process ranks: messages
travel as ``isend`` / ``irecv`` on the enclosing group, so no two-rank process group is created per edge (the
reference emulates p2p with a broadcast inside a 2-rank group, which costs one communicator per edge).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from math import log as mlog
from typing import List, Optional, Tuple


class Edge:
    def __init__(self, local_master_rank: int, dest: int, src: int, local_rank: int) -> None:
        self.src = src
        self.dest = dest
        self.process_group = None  # kept for API compatibility; p2p needs no group of its own

    def __repr__(self) -> str:
        return f"Edge({self.src}->{self.dest})"


class GraphManager(ABC):
    def __init__(self, rank: int, world_size: int, nprocs_per_node: int = 1, local_rank: int = 0, peers_per_itr: int = 1) -> None:
        assert int(peers_per_itr) >= 1
        self.rank = rank
        self.world_size = world_size
        self.phone_book: List[List[Edge]] = [[] for _ in range(world_size)]
        self._peers_per_itr = peers_per_itr
        self._group_indices = list(range(peers_per_itr))
        self.nprocs_per_node = nprocs_per_node
        self.local_rank = local_rank
        self._make_graph()

    @property
    def peers_per_itr(self) -> int:
        return self._peers_per_itr

    @peers_per_itr.setter
    def peers_per_itr(self, v: int) -> None:
        self._peers_per_itr = v
        self._group_indices = list(range(v))

    @abstractmethod
    def _make_graph(self) -> None:
        """Fill ``phone_book[r]`` with the ordered out-edges of every logical rank ``r``."""

    def _add_peers(self, rank: int, peers: List[int]) -> None:
        known = {e.dest for e in self.phone_book[rank]}
        for peer in peers:
            dest = peer * self.nprocs_per_node
            if dest not in known:
                known.add(dest)
                self.phone_book[rank].append(Edge(self.rank * self.nprocs_per_node, dest, rank * self.nprocs_per_node, self.local_rank))

    @abstractmethod
    def is_regular_graph(self) -> bool:
        """Every node has as many in-peers as out-peers."""

    @abstractmethod
    def is_bipartite_graph(self) -> bool:
        ...

    @abstractmethod
    def is_passive(self, rank: Optional[int] = None) -> bool:
        ...

    @abstractmethod
    def is_dynamic_graph(self) -> bool:
        """Out-peers rotate from one iteration to the next."""

    def get_edges(self, rotate: bool = False) -> Tuple[List[Edge], List[Edge]]:
        """(out-edges, in-edges) of this rank for the current iteration."""
        if rotate:
            self._rotate_group_indices()
        out_edges, in_edges = [], []
        me = self.rank * self.nprocs_per_node
        for gi in self._group_indices:
            out_edges.append(self.phone_book[self.rank][gi])
            for r, edges in enumerate(self.phone_book):
                if r != self.rank and gi < len(edges) and edges[gi].dest == me:
                    in_edges.append(edges[gi])
        return out_edges, in_edges

    def get_peers(self, rotate: bool = False) -> Tuple[List[int], List[int]]:
        out_edges, in_edges = self.get_edges(rotate)
        return [e.dest for e in out_edges], [e.src // self.nprocs_per_node for e in in_edges]

    def _rotate_group_indices(self) -> None:
        n = len(self.phone_book[self.rank])
        self._group_indices = [(g + self.peers_per_itr) % n for g in self._group_indices]

    def _rotate_forward(self, r: int, p: int) -> int:
        return (r + p) % self.world_size

    def _rotate_backward(self, r: int, p: int) -> int:
        return (r - p) % self.world_size


class _Flags:
    regular, bipartite, dynamic = True, False, True

    def is_regular_graph(self) -> bool:
        return self.regular

    def is_bipartite_graph(self) -> bool:
        return self.bipartite

    def is_dynamic_graph(self) -> bool:
        return self.dynamic

    def is_passive(self, rank: Optional[int] = None) -> bool:
        if not self.bipartite:
            return False
        rank = self.rank if rank is None else rank  # type: ignore[attr-defined]
        return rank % 2 == 0


def _hops_exp(world: int, base: int = 2) -> range:
    return range(0, int(mlog(world - 1, base)) + 1) if world > 2 else range(0, 1)


class DynamicDirectedExponentialGraph(_Flags, GraphManager):
    """Peers at distance +-2^i."""

    def _make_graph(self) -> None:
        for r in range(self.world_size):
            for i in _hops_exp(self.world_size):
                self._add_peers(r, [self._rotate_forward(r, 2**i), self._rotate_backward(r, 2**i)])


class NPeerDynamicDirectedExponentialGraph(_Flags, GraphManager):
    """``peers_per_itr`` forward peers at distances j * (n+1)^i."""

    def _make_graph(self) -> None:
        n = self._peers_per_itr
        for r in range(self.world_size):
            for i in _hops_exp(self.world_size, n + 1):
                for j in range(1, n + 1):
                    self._add_peers(r, [self._rotate_forward(r, j * (n + 1) ** i)])


class _BipartiteMixin(_Flags):
    bipartite = True

    def _add_if_alternating(self, r: int, f: int, b: int) -> None:
        if not self.is_passive(r) and self.is_passive(f) and self.is_passive(b):
            self._add_peers(r, [f, b])  # type: ignore[attr-defined]
        elif self.is_passive(r) and not (self.is_passive(f) or self.is_passive(b)):
            self._add_peers(r, [f, b])  # type: ignore[attr-defined]


class DynamicBipartiteExponentialGraph(_BipartiteMixin, GraphManager):
    def _make_graph(self) -> None:
        for r in range(self.world_size):
            for i in _hops_exp(self.world_size):
                d = 1 if i == 0 else 1 + 2**i
                self._add_if_alternating(r, self._rotate_forward(r, d), self._rotate_backward(r, d))


class DynamicDirectedLinearGraph(_Flags, GraphManager):
    def _make_graph(self) -> None:
        for r in range(self.world_size):
            for i in range(1, self.world_size, 2):
                self._add_peers(r, [self._rotate_forward(r, i), self._rotate_backward(r, i)])


class DynamicBipartiteLinearGraph(_BipartiteMixin, GraphManager):
    def _make_graph(self) -> None:
        for r in range(self.world_size):
            for i in range(1, self.world_size):
                self._add_if_alternating(r, self._rotate_forward(r, i), self._rotate_backward(r, i))


class RingGraph(_Flags, GraphManager):
    dynamic = False

    def _make_graph(self) -> None:
        for r in range(self.world_size):
            self._add_peers(r, [self._rotate_forward(r, 1), self._rotate_backward(r, 1)])
