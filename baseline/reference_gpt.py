"""The reference arm's model: a plain torch.nn pre-LN GPT wrapped by the UNMODIFIED reference library
(fairscale from baseline/_ref): its FullyShardedDataParallel and checkpoint_wrapper, stock code paths.

Nothing from fairscale_b200 is imported here. GEMMs run on cuBLAS, attention on torch's
scaled_dot_product_attention, collectives on NCCL.
"""

import torch
from torch import nn
from torch.nn import functional as F


class RefBlock(nn.Module):
    def __init__(self, d, heads, ffn):
        super().__init__()
        self.heads = heads
        self.ln1 = nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)
        self.ln2 = nn.LayerNorm(d)
        self.fc1 = nn.Linear(d, ffn)
        self.fc2 = nn.Linear(ffn, d)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, s, d))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


class RefEmbed(nn.Module):
    def __init__(self, vocab, d, seq):
        super().__init__()
        self.wte = nn.Embedding(vocab, d)
        self.wpe = nn.Embedding(seq, d)

    def forward(self, tokens):
        return self.wte(tokens) + self.wpe(torch.arange(tokens.shape[1], device=tokens.device))


class RefHead(nn.Module):
    def __init__(self, vocab, d):
        super().__init__()
        self.ln_f = nn.LayerNorm(d)
        self.out = nn.Linear(d, vocab, bias=False)

    def forward(self, x):
        return self.out(self.ln_f(x))


class RefGPT(nn.Module):
    def __init__(self, embed, blocks, head):
        super().__init__()
        self.embed = embed
        self.blocks = nn.ModuleList(blocks)
        self.head = head

    def forward(self, tokens):
        x = self.embed(tokens)
        for b in self.blocks:
            x = b(x)
        return self.head(x)


def build_reference_fsdp_gpt(vocab, d, heads, layers, ffn, seq, device):
    from fairscale.nn import FullyShardedDataParallel as FSDP
    from fairscale.nn import checkpoint_wrapper

    kw = dict(mixed_precision=True, compute_dtype=torch.bfloat16, reshard_after_forward=True, flatten_parameters=True)

    def init(m):
        for p in m.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, 0.0, 0.02)
        return m

    embed = FSDP(init(RefEmbed(vocab, d, seq)).to(device), **kw)
    blocks = [FSDP(checkpoint_wrapper(init(RefBlock(d, heads, ffn)).to(device)), **kw) for _ in range(layers)]
    head = FSDP(init(RefHead(vocab, d)).to(device), **kw)
    return FSDP(RefGPT(embed, blocks, head), **kw)
