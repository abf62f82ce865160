"""Mixing weights of gossip averaging (interface of .../gossip/mixing_manager.py:18-59).

A mixing manager answers two questions about one node of the communication graph: with which weights does it combine its
own value and what it sends to its out-peers, and does that choice keep the push-sum weight at 1 (``is_regular``: a
regular graph mixed uniformly has a uniform stationary distribution, so no de-biasing is needed).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Dict, Optional, Union

import torch

from .graph_manager import GraphManager

Weights = Dict[Union[str, int], torch.Tensor]


class MixingManager(ABC):
    def __init__(self, graph: GraphManager, device: Optional[torch.device]) -> None:
        self.graph_manager = graph
        self.device = device

    @abstractmethod
    def is_uniform(self) -> bool:
        """Do all out-going messages (and the kept share) carry the same weight?"""

    @abstractmethod
    def get_mixing_weights(self, residual_adjusted: bool = True) -> Weights:
        """``{"lo": kept share, "uniform": ..., peer: weight of the message to peer, ...}`` as 1-element tensors."""

    def is_regular(self) -> bool:
        return self.is_uniform() and self.graph_manager.is_regular_graph()


class UniformMixing(MixingManager):
    """The node and each of its ``d`` out-peers get ``1 / (d + 1)``.  With ``residual_adjusted`` the messages carry weight 1
    instead, because the sender multiplies by the kept share itself before it sends."""

    def is_uniform(self) -> bool:
        return True

    def get_mixing_weights(self, residual_adjusted: bool = True) -> Weights:
        out_peers, _ = self.graph_manager.get_peers()
        share = 1.0 / (len(out_peers) + 1.0)
        message = 1.0 if residual_adjusted else share

        def one(value: float) -> torch.Tensor:
            return torch.tensor([value], device=self.device)

        weights: Weights = {"lo": one(share), "uniform": one(message)}
        weights.update({peer: one(message) for peer in out_peers})
        return weights
