"""Small reference models shared by tests (plain torch.nn, CPU friendly)."""
import torch
from torch import nn


class TinyDecoderLM(nn.Module):
    """Pre-LayerNorm decoder-only LM: vocab 10000, d_model 256, 4 heads, 2 layers, FFN 1024 GELU by default."""

    def __init__(self, vocab=10000, d_model=256, heads=4, layers=2, ffn=1024, max_seq=64):
        super().__init__()
        self.tok = nn.Embedding(vocab, d_model)
        self.pos = nn.Embedding(max_seq, d_model)
        self.blocks = nn.ModuleList([_Block(d_model, heads, ffn) for _ in range(layers)])
        self.ln_f = nn.LayerNorm(d_model)
        self.head = nn.Linear(d_model, vocab, bias=False)
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, 0.0, 0.02)

    def forward(self, tokens):
        b, s = tokens.shape
        h = self.tok(tokens) + self.pos(torch.arange(s, device=tokens.device))
        for blk in self.blocks:
            h = blk(h)
        return self.head(self.ln_f(h))


class _Block(nn.Module):
    def __init__(self, d, heads, ffn):
        super().__init__()
        self.ln1 = nn.LayerNorm(d)
        self.ln2 = nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)
        self.fc1 = nn.Linear(d, ffn)
        self.fc2 = nn.Linear(ffn, d)
        self.heads = heads

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, s, d))
        return x + self.fc2(nn.functional.gelu(self.fc1(self.ln2(x))))


def lm_loss(logits, tokens):
    """Next-token cross entropy: targets are the inputs shifted by one."""
    return nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.size(-1)), tokens[:, 1:].reshape(-1))
