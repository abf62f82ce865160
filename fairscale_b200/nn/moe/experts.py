"""Local experts of an MoE layer held as stacked weights, so that all of them run in one grouped GEMM launch.

The reference keeps a ``ModuleList`` of feed-forward modules and loops over them in Python
(fairscale/nn/moe/moe_layer.py:83-85); with 8 local experts of 2048 tokens each that is 16 small GEMM launches per
layer and direction.  ``GroupedExperts`` is a drop-in ``experts`` argument of :class:`MOELayer`: the layer hands it the
whole ``[local experts, tokens, model]`` block at once.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from ...ops.gemm import grouped_mlp


class GroupedExperts(nn.Module):
    """``num_local_experts`` GELU feed-forward experts ``model_dim -> hidden_dim -> model_dim`` with biases."""

    grouped = True

    def __init__(self, num_local_experts: int, model_dim: int, hidden_dim: int) -> None:
        super().__init__()
        self.num_local_experts = num_local_experts
        self.w1 = nn.Parameter(torch.empty(num_local_experts, hidden_dim, model_dim))
        self.b1 = nn.Parameter(torch.zeros(num_local_experts, hidden_dim))
        self.w2 = nn.Parameter(torch.empty(num_local_experts, model_dim, hidden_dim))
        self.b2 = nn.Parameter(torch.zeros(num_local_experts, model_dim))
        for w in (self.w1, self.w2):
            for e in range(num_local_experts):  # same initialisation as nn.Linear, expert by expert
                nn.init.kaiming_uniform_(w[e], a=math.sqrt(5))
        for p in self.parameters():
            p.expert = True  # type: ignore[attr-defined]

    def __len__(self) -> int:
        return self.num_local_experts

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # x: [E_local, tokens, model_dim]
        return grouped_mlp(x, self.w1, self.b1, self.w2, self.b2)
