"""Mixing weights of gossip averaging (parity: .../gossip/mixing_manager.py:18-59)."""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Dict, Optional, Union

import torch

from .graph_manager import GraphManager


class MixingManager(ABC):
    def __init__(self, graph: GraphManager, device: Optional[torch.device]) -> None:
        self.graph_manager = graph
        self.device = device

    def is_regular(self) -> bool:
        """No bias accumulates in the local entry of the stationary distribution (push-sum weight stays 1)."""
        return self.graph_manager.is_regular_graph() and self.is_uniform()

    @abstractmethod
    def is_uniform(self) -> bool:
        ...

    @abstractmethod
    def get_mixing_weights(self, residual_adjusted: bool = True) -> Dict[Union[str, int], torch.Tensor]:
        ...


class UniformMixing(MixingManager):
    """Every out-peer and the node itself get weight 1 / (out-degree + 1)."""

    def get_mixing_weights(self, residual_adjusted: bool = True) -> Dict[Union[str, int], torch.Tensor]:
        out_peers, _ = self.graph_manager.get_peers()
        lo = torch.tensor([1.0 / (len(out_peers) + 1.0)], device=self.device)
        w = lo / lo if residual_adjusted else lo  # residual-adjusted: the local weight is applied afterwards
        weights: Dict[Union[str, int], torch.Tensor] = {"lo": lo.clone(), "uniform": w.clone()}
        for p in out_peers:
            weights[p] = w.clone()
        return weights

    def is_uniform(self) -> bool:
        return True
