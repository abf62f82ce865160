"""Mixture-of-experts GPT: the flagship pre-LN block with every other feed-forward replaced by a top-2 MoE layer.

Expert-parallel configuration of the reference's MOELayer / Top2Gate (fairscale/nn/moe/moe_layer.py:23-91): the dense
parts are replicated (data parallel), each rank owns ``num_local_experts`` GELU experts held as stacked weights
(``GroupedExperts``: one grouped tcgen05 launch for all of them), tokens travel to their experts with the NVLink row
scatter / gather kernels when a workspace exists for the expert group (NCCL all-to-all otherwise), and routing uses
the index kernels of ``csrc/top2gate.cu``.  ``forward(tokens, targets)`` returns ``loss + aux_weight * sum(l_aux)``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..nn.moe import GroupedExperts, MOELayer, Top2Gate
from ..ops.attention import causal_attention
from ..ops.gemm import linear
from ..ops.norm import LayerNorm
from .gpt import Block, Embedding, GPTConfig, Head


@dataclass
class MoELMConfig(GPTConfig):
    vocab_size: int = 32000
    d_model: int = 1024
    n_heads: int = 16
    n_layers: int = 12
    ffn: int = 4096
    max_seq: int = 1024
    num_local_experts: int = 8
    moe_every: int = 2          # every `moe_every`-th block carries the MoE feed-forward
    aux_weight: float = 0.01


class MoEBlock(nn.Module):
    """Attention as in :class:`Block`; the feed-forward is ``x + MoE(LN(x))``."""

    def __init__(self, cfg: MoELMConfig, group: Any = None):
        super().__init__()
        d = cfg.d_model
        self.n_heads = cfg.n_heads
        self.ln1 = LayerNorm(d, cfg.ln_eps)
        self.qkv_w = nn.Parameter(torch.empty(3 * d, d))
        self.qkv_b = nn.Parameter(torch.zeros(3 * d))
        self.proj_w = nn.Parameter(torch.empty(d, d))
        self.proj_b = nn.Parameter(torch.zeros(d))
        self.ln2 = LayerNorm(d, cfg.ln_eps)
        for w in (self.qkv_w, self.proj_w):
            nn.init.normal_(w, 0.0, cfg.init_std)
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        gate = Top2Gate(d, cfg.num_local_experts * world)
        nn.init.normal_(gate.wg.weight, 0.0, cfg.init_std)
        self.moe = MOELayer(gate, GroupedExperts(cfg.num_local_experts, d, cfg.ffn), group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.ln1(x)
        a = causal_attention(linear(h, self.qkv_w, self.qkv_b), self.n_heads)
        x = linear(a, self.proj_w, self.proj_b, residual=x)
        return x + self.moe(self.ln2(x))


class MoELM(nn.Module):
    def __init__(self, cfg: MoELMConfig, group: Any = None):
        super().__init__()
        self.cfg = cfg
        self.embed = Embedding(cfg)
        self.blocks = nn.ModuleList(
            [MoEBlock(cfg, group) if (i % cfg.moe_every) == cfg.moe_every - 1 else Block(cfg) for i in range(cfg.n_layers)])
        self.head = Head(cfg)

    def expert_parameters(self):
        return [p for p in self.parameters() if getattr(p, "expert", False)]

    def dense_parameters(self):
        return [p for p in self.parameters() if not getattr(p, "expert", False)]

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.embed(tokens)
        aux = None
        for blk in self.blocks:
            x = blk(x)
            if isinstance(blk, MoEBlock):
                aux = blk.moe.l_aux if aux is None else aux + blk.moe.l_aux
        out = self.head(x, targets)
        if targets is not None and aux is not None:
            out = out + self.cfg.aux_weight * aux.to(out.dtype)
        return out
