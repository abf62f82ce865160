"""Tensor-parallel Llama-style language model (RMSNorm, RoPE, SwiGLU) on the model_parallel layers.

The model family of the reference's Megatron-style layers (fairscale/nn/model_parallel/layers.py): QKV and gate/up
projections are ``ColumnParallelLinear`` (heads / hidden units split over the model-parallel group), the output and down
projections are ``RowParallelLinear``, the token table is a ``VocabParallelEmbedding`` and the loss is
``vocab_parallel_cross_entropy`` over vocabulary-sharded logits.

Between the parallel linears the activations are *sequence-parallel*: each rank holds ``tokens / world`` rows, the
column-parallel layers take them through the fused all-gather->GEMM kernel and the row-parallel layers return them
through the fused GEMM->reduce-scatter kernel (``sequence_parallel=True``), so a block issues no stand-alone
collective and the norms / residual adds run on 1 / world of the tokens.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch
from torch import nn

from ..nn.model_parallel import (
    ColumnParallelLinear,
    RowParallelLinear,
    VocabParallelEmbedding,
    get_model_parallel_group,
    get_model_parallel_world_size,
    vocab_parallel_cross_entropy,
)
from ..ops.activations import swiglu
from ..ops.attention import causal_attention
from ..ops.norm import RMSNorm
from ..ops.rope import rope_qkv
from ..parallel import comm


@dataclass
class TPLlamaConfig:
    vocab_size: int = 32000
    d_model: int = 4096
    n_heads: int = 32
    n_layers: int = 32
    ffn: int = 11008
    max_seq: int = 4096
    rope_theta: float = 10000.0
    init_std: float = 0.02

    @classmethod
    def tiny(cls, **kw: Any) -> "TPLlamaConfig":
        base = dict(vocab_size=256, d_model=32, n_heads=4, n_layers=2, ffn=64, max_seq=16)
        base.update(kw)
        return cls(**base)


class _ScatterRows(torch.autograd.Function):
    """Full ``[T, D]`` (identical on every rank) -> this rank's ``T / world`` rows; backward all-gathers the row gradients."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, group: Any) -> torch.Tensor:  # type: ignore[override]
        ctx.group = group
        w, r = comm.group_size(group), comm.group_rank(group)
        n = x.shape[0] // w
        return x[r * n : (r + 1) * n].contiguous()

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> Any:  # type: ignore[override]
        w = comm.group_size(ctx.group)
        out = torch.empty((g.shape[0] * w,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        comm.all_gather_into(out.view(-1), g.contiguous().view(-1), group=ctx.group)
        return out, None


class _GatherRows(torch.autograd.Function):
    """This rank's rows -> full ``[T, D]`` on every rank.  The consumer (a column-parallel linear entered through
    ``copy_to_model_parallel_region``) already sums its input gradient over the group, so the incoming gradient is the
    complete one on every rank and backward only keeps this rank's rows."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, group: Any) -> torch.Tensor:  # type: ignore[override]
        ctx.group = group
        w = comm.group_size(group)
        out = torch.empty((x.shape[0] * w,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        comm.all_gather_into(out.view(-1), x.contiguous().view(-1), group=group)
        return out

    @staticmethod
    def backward(ctx: Any, g: torch.Tensor) -> Any:  # type: ignore[override]
        w, r = comm.group_size(ctx.group), comm.group_rank(ctx.group)
        n = g.shape[0] // w
        return g[r * n : (r + 1) * n].contiguous(), None


class TPBlock(nn.Module):
    def __init__(self, cfg: TPLlamaConfig):
        super().__init__()
        init = lambda w: nn.init.normal_(w, std=cfg.init_std)  # noqa: E731
        world = get_model_parallel_world_size()
        assert cfg.n_heads % world == 0
        self.cfg = cfg
        self.local_heads = cfg.n_heads // world
        self.norm1 = RMSNorm(cfg.d_model)
        # stride=3 / stride=2: every rank receives its slice of q, k, v (of gate, up) rather than a slice of the concatenation
        self.qkv = ColumnParallelLinear(cfg.d_model, 3 * cfg.d_model, bias=False, gather_output=False, init_method=init, stride=3,
                                        sequence_parallel=True)
        self.proj = RowParallelLinear(cfg.d_model, cfg.d_model, bias=False, input_is_parallel=True, init_method=init, sequence_parallel=True)
        self.norm2 = RMSNorm(cfg.d_model)
        self.gate_up = ColumnParallelLinear(cfg.d_model, 2 * cfg.ffn, bias=False, gather_output=False, init_method=init, stride=2,
                                            sequence_parallel=True)
        self.down = RowParallelLinear(cfg.ffn, cfg.d_model, bias=False, input_is_parallel=True, init_method=init, sequence_parallel=True)

    def forward(self, x: torch.Tensor, batch: int) -> torch.Tensor:  # x: [T / world, D], rows in (batch, seq) order
        cfg = self.cfg
        qkv = self.qkv(self.norm1(x))  # [T, 3 * D / world]
        S = qkv.shape[0] // batch
        qkv = rope_qkv(qkv.view(batch, S, 3, self.local_heads, cfg.d_model // cfg.n_heads), cfg.rope_theta)
        o = causal_attention(qkv.reshape(batch, S, -1), self.local_heads)
        x = x + self.proj(o.reshape(batch * S, -1))
        return x + self.down(swiglu(self.gate_up(self.norm2(x))))


class TPLlama(nn.Module):
    """``forward(tokens[B, S], targets[B, S]) -> mean loss``; with ``targets=None`` returns the vocabulary-sharded logits."""

    def __init__(self, cfg: TPLlamaConfig):
        super().__init__()
        self.cfg = cfg
        init = lambda w: nn.init.normal_(w, std=cfg.init_std)  # noqa: E731
        self.embed = VocabParallelEmbedding(cfg.vocab_size, cfg.d_model, init_method=init)
        self.blocks = nn.ModuleList([TPBlock(cfg) for _ in range(cfg.n_layers)])
        self.norm = RMSNorm(cfg.d_model)
        self.head = ColumnParallelLinear(cfg.d_model, cfg.vocab_size, bias=False, gather_output=False, init_method=init)

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None) -> torch.Tensor:
        group = get_model_parallel_group()
        B, S = tokens.shape
        x = self.embed(tokens).reshape(B * S, -1)
        x = _ScatterRows.apply(x, group)
        for blk in self.blocks:
            x = blk(x, B)
        x = _GatherRows.apply(self.norm(x), group)
        logits = self.head(x)  # [T, V / world]
        if targets is None:
            return logits
        return vocab_parallel_cross_entropy(logits.float(), targets.reshape(-1)).mean()
