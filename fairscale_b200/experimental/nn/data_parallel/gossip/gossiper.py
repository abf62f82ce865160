"""Gossip averaging steps: push-sum (directed) and push-pull (doubly stochastic).

Capability parity with fairscale/experimental/nn/data_parallel/gossip/gossiper.py:30-280.  One ``mix`` posts all
sends and receives of the iteration as a single batch of p2p operations and waits once, instead of one blocking
broadcast per edge.
"""

from __future__ import annotations

import logging
from typing import Any, Iterator, Optional, Tuple

from enum import Enum

import torch
import torch.distributed as dist

from .graph_manager import GraphManager
from .mixing_manager import MixingManager, UniformMixing


class dist_backend(str, Enum):
    """Names of the process-group backends the gossip code distinguishes."""

    UNDEFINED = "undefined"
    TCP = "tcp"
    MPI = "mpi"
    GLOO = "gloo"
    NCCL = "nccl"


class Gossiper:
    def __init__(self, msg: torch.Tensor, graph: GraphManager, device: Optional[torch.device] = None,
                 mixing: Optional[MixingManager] = None, logger: Optional[logging.Logger] = None,
                 rank: Optional[int] = None, world_size: Optional[int] = None, group: Any = None) -> None:
        self.logger = logger
        if rank is None or world_size is None:
            assert dist.is_initialized()
            rank, world_size = dist.get_rank(), dist.get_world_size()
        self.rank, self.world_size, self.group = rank, world_size, group
        assert isinstance(graph, GraphManager)
        self._graph_manager = graph
        self.device = device if device is not None else msg.device
        self.passive = graph.is_passive()
        self.refresh_peers_(rotate=False)
        self._mixing_manager = mixing if mixing is not None else UniformMixing(graph, self.device)
        self.refresh_mixing_weights_()
        self.regular = self._mixing_manager.is_regular()
        self._ps_weight = torch.ones(1, dtype=msg.dtype, device=self.device)
        n = msg.numel() + (0 if self.regular else 1)
        self.in_msg_buffer = torch.zeros(n, dtype=msg.dtype, device=self.device)
        self.placeholder = torch.zeros_like(self.in_msg_buffer)

    @property
    def ps_weight(self) -> torch.Tensor:
        return self._ps_weight

    @ps_weight.setter
    def ps_weight(self, v: torch.Tensor) -> None:
        self._ps_weight.data[0] = v

    @property
    def peers_per_itr(self) -> int:
        return self._graph_manager.peers_per_itr

    @peers_per_itr.setter
    def peers_per_itr(self, v: int) -> None:
        self._graph_manager.peers_per_itr = v

    def refresh_peers_(self, rotate: Optional[bool] = None) -> None:
        if rotate is None:
            rotate = self._graph_manager.is_dynamic_graph()
        assert not (rotate and not self._graph_manager.is_dynamic_graph())
        self.out_edges, self.in_edges = self._graph_manager.get_edges(rotate)

    def refresh_mixing_weights_(self, residual_adjusted: bool = False) -> None:
        self.mixing_weights = self._mixing_manager.get_mixing_weights(residual_adjusted)

    def mix_out_msg_(self, out_msg: torch.Tensor, ps_weight: torch.Tensor) -> Iterator[torch.Tensor]:
        """Messages for the out-edges, weighted on the fly."""
        self.refresh_mixing_weights_(residual_adjusted=True)
        self.ps_weight = ps_weight
        if not self.regular:
            out_msg = torch.cat([out_msg, self.ps_weight.to(out_msg.dtype)])
        if self._mixing_manager.is_uniform():
            out_msg = out_msg * self.mixing_weights["uniform"].to(out_msg.dtype)
            for _ in self.out_edges:
                yield out_msg
        else:
            for e in self.out_edges:
                yield out_msg * self.mixing_weights[e.dest].to(out_msg.dtype)

    def parse_in_msg_buffer(self) -> Tuple[torch.Tensor, torch.Tensor]:
        msg = self.in_msg_buffer
        if not self.regular:
            return msg[:-1], msg[-1]
        return msg, self.ps_weight * self.peers_per_itr

    def _exchange(self, out_msg: torch.Tensor, ps_weight: torch.Tensor) -> None:
        msgs = list(self.mix_out_msg_(out_msg, ps_weight))
        recv_bufs = [self.in_msg_buffer] if len(self.in_edges) == 1 else [torch.empty_like(self.in_msg_buffer) for _ in self.in_edges]
        ops = [dist.P2POp(dist.isend, m.contiguous(), e.dest, self.group) for m, e in zip(msgs, self.out_edges)]
        ops += [dist.P2POp(dist.irecv, b, e.src, self.group) for b, e in zip(recv_bufs, self.in_edges)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        if len(self.in_edges) != 1:
            self.in_msg_buffer.zero_()
            for b in recv_bufs:
                self.in_msg_buffer.add_(b)

    def mix(self, out_msg: torch.Tensor, ps_weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """One gossip step: returns (sum of incoming messages, incoming push-sum weight)."""
        assert out_msg.device.type == self.device.type
        self._exchange(out_msg, ps_weight)
        self.refresh_peers_()
        return self.parse_in_msg_buffer()

    def clean_msg_buffers_(self) -> None:
        """Nothing is left in flight after ``mix`` returns."""


class PushSum(Gossiper):
    """Push-sum consensus: column-stochastic mixing, de-biased by the push-sum weight."""


class PushPull(Gossiper):
    """Doubly stochastic consensus over symmetric (bipartite) exchanges; same wire protocol as push-sum since
    sends and receives of one iteration are posted together."""
