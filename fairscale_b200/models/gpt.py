"""GPT-style decoder-only language model built on this library's fused ops.

Architecture (pre-LayerNorm, learned positions, GELU feed-forward, untied output head) follows the
flagship FSDP configuration: 24 layers, d_model 2048, 16 heads, FFN 8192, vocab 50304, seq 2048.
Every block is 7 kernel launches forward: LN, QKV GEMM(+bias), attention, proj GEMM(+bias+residual),
LN, FC1 GEMM(+bias+GELU), FC2 GEMM(+bias+residual).

The reference's benchmark model is ``benchmarks/models/transformer_lm.py:16-207`` (post-LN,
``nn.MultiheadAttention``, ReLU/GELU FFN); this one is the pre-LN GPT the target configuration names.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch
from torch import nn

from ..ops.attention import causal_attention
from ..ops.embedding import embedding
from ..ops.gemm import linear
from ..ops.loss import cross_entropy
from ..ops.mlp import mlp
from ..ops.norm import LayerNorm


@dataclass
class GPTConfig:
    vocab_size: int = 50304
    d_model: int = 2048
    n_heads: int = 16
    n_layers: int = 24
    ffn: int = 8192
    max_seq: int = 2048
    init_std: float = 0.02
    ln_eps: float = 1e-5

    @staticmethod
    def gpt_1p3b() -> "GPTConfig":
        return GPTConfig()

    @staticmethod
    def tiny(vocab: int = 512, d_model: int = 128, n_heads: int = 2, n_layers: int = 2, ffn: int = 512, max_seq: int = 128) -> "GPTConfig":
        return GPTConfig(vocab, d_model, n_heads, n_layers, ffn, max_seq)

    def num_params(self) -> int:
        per_block = 4 * self.d_model * self.d_model + 2 * self.d_model * self.ffn + 9 * self.d_model + self.ffn
        return self.n_layers * per_block + (2 * self.vocab_size + self.max_seq + 2) * self.d_model

    def flops_per_token(self, seq: int, with_recompute: bool = True) -> float:
        """Training FLOPs per token: 6 x matmul parameters (+2 x for activation recomputation) + causal attention."""
        matmul_params = self.n_layers * (4 * self.d_model**2 + 2 * self.d_model * self.ffn) + self.vocab_size * self.d_model
        factor = 8.0 if with_recompute else 6.0
        block_params = matmul_params - self.vocab_size * self.d_model
        attn = self.n_layers * 2 * 2 * seq * self.d_model / 2  # QK^T and PV, causal half
        return 6.0 * self.vocab_size * self.d_model + factor * block_params + (factor / 2.0) * attn


class Embedding(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.wte = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model))
        self.wpe = nn.Parameter(torch.empty(cfg.max_seq, cfg.d_model))
        nn.init.normal_(self.wte, 0.0, cfg.init_std)
        nn.init.normal_(self.wpe, 0.0, cfg.init_std)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return embedding(tokens, self.wte, self.wpe)


class Block(nn.Module):
    # The first use of this block's matrices is the QKV ``linear`` (the LayerNorm before it only reads small parameters),
    # so an FSDP unit wrapping one block may fuse its parameter all-gather into that product (FSB200_FSDP_AG_GEMM=1).
    fsb_fused_first_gemm = True

    def __init__(self, cfg: GPTConfig):
        super().__init__()
        d, f = cfg.d_model, cfg.ffn
        self.n_heads = cfg.n_heads
        self.ln1 = LayerNorm(d, cfg.ln_eps)
        self.qkv_w = nn.Parameter(torch.empty(3 * d, d))
        self.qkv_b = nn.Parameter(torch.zeros(3 * d))
        self.proj_w = nn.Parameter(torch.empty(d, d))
        self.proj_b = nn.Parameter(torch.zeros(d))
        self.ln2 = LayerNorm(d, cfg.ln_eps)
        self.fc1_w = nn.Parameter(torch.empty(f, d))
        self.fc1_b = nn.Parameter(torch.zeros(f))
        self.fc2_w = nn.Parameter(torch.empty(d, f))
        self.fc2_b = nn.Parameter(torch.zeros(d))
        for w in (self.qkv_w, self.proj_w, self.fc1_w, self.fc2_w):
            nn.init.normal_(w, 0.0, cfg.init_std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.ln1(x)
        qkv = linear(h, self.qkv_w, self.qkv_b)
        a = causal_attention(qkv, self.n_heads)
        x = linear(a, self.proj_w, self.proj_b, residual=x)
        h = self.ln2(x)
        return mlp(h, self.fc1_w, self.fc1_b, self.fc2_w, self.fc2_b, residual=x)


class Head(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.ln_f = LayerNorm(cfg.d_model, cfg.ln_eps)
        self.weight = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model))
        nn.init.normal_(self.weight, 0.0, cfg.init_std)

    def forward(self, x: torch.Tensor, targets: Optional[torch.Tensor] = None) -> torch.Tensor:
        logits = linear(self.ln_f(x), self.weight)
        if targets is None:
            return logits
        return cross_entropy(logits, targets)


class GPT(nn.Module):
    """``forward(tokens, targets)`` returns the mean next-token loss (or logits when ``targets`` is None)."""

    def __init__(self, cfg: GPTConfig, wrap_block: Optional[Callable[[nn.Module], nn.Module]] = None,
                 wrap_unit: Optional[Callable[[nn.Module], nn.Module]] = None):
        super().__init__()
        self.cfg = cfg
        wb = wrap_block or (lambda m: m)
        wu = wrap_unit or (lambda m: m)
        self.embed = wu(Embedding(cfg))
        self.blocks = nn.ModuleList([wb(Block(cfg)) for _ in range(cfg.n_layers)])
        self.head = wu(Head(cfg))

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.embed(tokens)
        for blk in self.blocks:
            x = blk(x)
        return self.head(x, targets)


def build_fsdp_gpt(cfg: GPTConfig, device: torch.device, process_group: Any = None, *, checkpoint_blocks: bool = True,
                   compute_dtype: torch.dtype = torch.bfloat16, nvlink_heap: bool = True, **fsdp_kwargs: Any) -> nn.Module:
    """The flagship training setup: every block is ``FSDP(checkpoint_wrapper(block))``, embedding and head are
    their own FSDP units, and a root FSDP ties them together (full shard, bf16 compute, fp32 master shards)."""
    from ..nn.checkpoint import checkpoint_wrapper
    from ..nn.data_parallel import FullyShardedDataParallel as FSDP

    from ..internal.parallel import ProcessGroupName, get_process_group_cached
    from ..parallel import nvlink, symm

    if process_group is None:
        process_group = get_process_group_cached()
    world = process_group.size()
    if nvlink_heap and world > 1 and device.type == "cuda" and nvlink.available() and symm.workspace_for(process_group) is None:
        # the compute-dtype shards live in the symmetric heap so peers all-gather them without staging
        # plus three rotating gradient windows (largest unit: the embedding / head matrix or one block), so that the
        # reduce-scatter kernels read the weight gradients where the GEMMs wrote them
        shard_mb = (2 * cfg.num_params() // world >> 20) + 64
        per_block = 4 * cfg.d_model * cfg.d_model + 2 * cfg.d_model * cfg.ffn + 9 * cfg.d_model + cfg.ffn
        unit = max((cfg.vocab_size + cfg.max_seq + 2) * cfg.d_model, per_block)  # embedding / head / one block
        window_bytes = 2 * unit + (1 << 20)
        ws = nvlink.enable(process_group, device, staging_mb=256, heap_mb=shard_mb + 3 * (window_bytes >> 20) + 8)
        ws.enable_grad_windows(window_bytes, count=3)
        symm.register_workspace(get_process_group_cached(ProcessGroupName.reduce_scatter), ws)

    kw = dict(process_group=process_group, mixed_precision=True, compute_dtype=compute_dtype, reshard_after_forward=True,
              flatten_parameters=True, compute_device=device, keep_low_precision_grads=True, persistent_compute_shards=True)
    kw.update(fsdp_kwargs)

    def wrap_block(m: nn.Module) -> nn.Module:
        m = m.to(device)
        if checkpoint_blocks:
            m = checkpoint_wrapper(m)
        return FSDP(m, **kw)

    def wrap_unit(m: nn.Module) -> nn.Module:
        return FSDP(m.to(device), **kw)

    model = GPT(cfg, wrap_block=wrap_block, wrap_unit=wrap_unit)
    return FSDP(model, **kw)
