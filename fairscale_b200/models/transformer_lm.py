"""The sequential GPT-2 style language model used by the pipeline / FSDP / MoE / offload benchmarks.

Same architecture and layer list as the reference's benchmark model (benchmarks/models/transformer_lm.py:16-207):
``Embedding * sqrt(d) -> sinusoidal positions (+dropout) -> N post-LN decoder layers (causal self-attention + ReLU
feed-forward or a top-2 MoE) -> Linear to the vocabulary``, as an ``nn.Sequential`` so that ``Pipe``, ``OffloadModel``
and ``auto_wrap`` can cut it anywhere.  Tokens are ``[batch, seq]``.  Attention goes through
:func:`fairscale_b200.ops.attention.causal_attention` (the tcgen05 flash kernels on bf16 CUDA tensors, PyTorch SDPA
otherwise) instead of ``nn.MultiheadAttention`` with a dense additive mask.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from ..nn.moe import MOELayer, Top2Gate
from ..ops.attention import causal_attention
from ..ops.dropout import Dropout


class EmbeddingLayer(nn.Embedding):
    def __init__(self, ntoken: int, ninp: int, initrange: float):
        super().__init__(ntoken, ninp)
        self.ninp_sqrt = math.sqrt(ninp)
        nn.init.uniform_(self.weight, -initrange, initrange)

    def forward(self, src: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        return super().forward(src) * self.ninp_sqrt


class PositionalEncodingLayer(nn.Module):
    def __init__(self, d_model: int, dropout: float = 0.1, max_len: int = 5000):
        super().__init__()
        self.dropout = Dropout(p=dropout)
        pos = torch.arange(max_len, dtype=torch.float32).unsqueeze(1)
        div = torch.exp(torch.arange(0, d_model, 2, dtype=torch.float32) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)
        self.register_buffer("pe", pe)

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # x: [B, S, D]
        return self.dropout(x + self.pe[: x.size(1)].to(x.dtype))


class FeedForwardLayer(nn.Module):
    def __init__(self, d_model: int, dim_feedforward: int, activation: Any, dropout: float) -> None:
        super().__init__()
        self.linear1 = nn.Linear(d_model, dim_feedforward)
        self.activation = activation
        self.dropout1 = Dropout(dropout)
        self.linear2 = nn.Linear(dim_feedforward, d_model)
        self.dropout2 = Dropout(dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dropout2(self.linear2(self.dropout1(self.activation(self.linear1(x)))))


class SelfAttention(nn.Module):
    """Packed-QKV causal attention (``in_proj`` then ``out_proj`` like ``nn.MultiheadAttention``)."""

    def __init__(self, d_model: int, nhead: int, dropout: float):
        super().__init__()
        assert d_model % nhead == 0
        self.nhead = nhead
        self.in_proj = nn.Linear(d_model, 3 * d_model)
        self.out_proj = nn.Linear(d_model, d_model)
        self.dropout = dropout

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, D = x.shape
        qkv = self.in_proj(x)  # [B, S, 3 * H * Dh], packed as (3, H, Dh)
        if self.dropout > 0 and self.training:
            q, k, v = (t.transpose(1, 2) for t in qkv.view(B, S, 3, self.nhead, D // self.nhead).unbind(2))
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, dropout_p=self.dropout).transpose(1, 2).reshape(B, S, D)
        else:
            o = causal_attention(qkv, self.nhead).reshape(B, S, D)
        return self.out_proj(o)


class TransformerDecoderLayer(nn.Module):
    def __init__(self, ninp: int, nhead: int, nhid: int, dropout: float, is_moe: bool = False, num_local_experts: int = 1,
                 norm_first: bool = False, layer_norm_eps: float = 1e-5, moe_group: Any = None):
        super().__init__()
        self.self_attn = SelfAttention(ninp, nhead, dropout)
        self.norm_first = norm_first
        self.norm1 = nn.LayerNorm(ninp, eps=layer_norm_eps)
        self.norm2 = nn.LayerNorm(ninp, eps=layer_norm_eps)
        self.dropout = Dropout(dropout)
        self.is_moe = is_moe
        if is_moe:
            world = dist.get_world_size(moe_group) if dist.is_initialized() else 1
            self.gate = Top2Gate(ninp, num_local_experts * world)
            experts = nn.ModuleList([FeedForwardLayer(ninp, nhid, nn.ReLU(), dropout) for _ in range(num_local_experts)])
            self.moe_layer = MOELayer(self.gate, experts, moe_group)
        else:
            self.ff_block = FeedForwardLayer(ninp, nhid, nn.ReLU(), dropout)

    def _ff(self, x: torch.Tensor) -> torch.Tensor:
        return self.moe_layer(x) if self.is_moe else self.ff_block(x)

    def forward(self, src: torch.Tensor) -> torch.Tensor:
        x = src
        if self.norm_first:
            x = x + self.dropout(self.self_attn(self.norm1(x)))
            return x + self._ff(self.norm2(x))
        x = self.norm1(x + self.dropout(self.self_attn(x)))
        return self.norm2(x + self._ff(x))


class LinearLayer(nn.Linear):
    def __init__(self, ninp: int, ntoken: int, initrange: float):
        super().__init__(ninp, ntoken)
        nn.init.zeros_(self.bias)
        nn.init.uniform_(self.weight, -initrange, initrange)


class TransformerLM(nn.Sequential):
    """``TransformerLM(ntokens, ninp, nhead, nhid, dropout, initrange, ndecoder, is_moe=False, num_local_experts=1)``."""

    def __init__(self, ntokens: int, ninp: int, nhead: int, nhid: int, dropout: float, initrange: float, ndecoder: int,
                 is_moe: bool = False, num_local_experts: int = 1, moe_group: Any = None):
        layers = [EmbeddingLayer(ntokens, ninp, initrange), PositionalEncodingLayer(ninp, dropout)]
        layers += [TransformerDecoderLayer(ninp, nhead, nhid, dropout, is_moe, num_local_experts, moe_group=moe_group) for _ in range(ndecoder)]
        layers.append(LinearLayer(ninp, ntokens, initrange))
        super().__init__(*layers)
