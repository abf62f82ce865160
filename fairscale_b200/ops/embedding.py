"""Token (+ learned position) embedding lookup and its scatter-add backward (``csrc/elementwise.cu``)."""

from __future__ import annotations

from typing import Optional

import torch

from . import _bind


def embedding_forward(tokens: torch.Tensor, wte: torch.Tensor, wpe: Optional[torch.Tensor] = None, scale: float = 1.0,
                      vocab_start: int = 0) -> torch.Tensor:
    """``wte[tokens - vocab_start] * scale (+ wpe[position])``; ids outside the local slice yield zeros."""
    H = wte.shape[1]
    seq = tokens.shape[-1]
    if not _bind.use_native(tokens, wte) or wte.dtype != torch.bfloat16 or H % 8:
        local = tokens - vocab_start
        inside = (local >= 0) & (local < wte.shape[0])
        out = torch.nn.functional.embedding(local.clamp(0, wte.shape[0] - 1), wte) * scale
        out = out * inside.unsqueeze(-1).to(out.dtype)
        if wpe is not None:
            out = out + wpe[:seq]
        return out
    tok = tokens.contiguous()
    out = torch.empty((*tokens.shape, H), dtype=wte.dtype, device=wte.device)
    _bind.call("fsb_embedding_fwd", tok.data_ptr(), wte.data_ptr(), _bind.ptr(wpe), out.data_ptr(), tok.numel(), H, seq,
               vocab_start, wte.shape[0], scale, _bind.stream_ptr(wte.device))
    return out


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, wte, wpe, scale: float, vocab_start: int):  # type: ignore[override]
        ctx.save_for_backward(tokens)
        ctx.shapes = (wte.shape, None if wpe is None else wpe.shape, wte.dtype)
        ctx.scale, ctx.vocab_start = scale, vocab_start
        return embedding_forward(tokens, wte, wpe, scale, vocab_start)

    @staticmethod
    def backward(ctx, dout):  # type: ignore[override]
        (tokens,) = ctx.saved_tensors
        wte_shape, wpe_shape, dtype = ctx.shapes
        H = wte_shape[1]
        seq = tokens.shape[-1]
        if not _bind.use_native(dout) or dout.dtype != torch.bfloat16 or H % 8:
            d = dout.reshape(-1, H).float()
            local = (tokens - ctx.vocab_start).reshape(-1)
            inside = (local >= 0) & (local < wte_shape[0])
            dwte = torch.zeros(wte_shape, dtype=torch.float32, device=dout.device)
            dwte.index_add_(0, local[inside], d[inside] * ctx.scale)
            dwpe = None
            if wpe_shape is not None:
                dwpe = torch.zeros(wpe_shape, dtype=torch.float32, device=dout.device)
                dwpe[:seq] = dout.reshape(-1, seq, H).float().sum(0)
                dwpe = dwpe.to(dtype)
            return None, dwte.to(dtype), dwpe, None, None
        d = dout.contiguous()
        dwte = torch.zeros(wte_shape, dtype=torch.float32, device=dout.device)
        dwpe = torch.zeros(wpe_shape, dtype=torch.float32, device=dout.device) if wpe_shape is not None else None
        _bind.call("fsb_embedding_bwd", tokens.contiguous().data_ptr(), d.data_ptr(), dwte.data_ptr(), _bind.ptr(dwpe), tokens.numel(),
                   H, seq, ctx.vocab_start, wte_shape[0], ctx.scale, _bind.stream_ptr(dout.device))
        return None, dwte.to(dtype), None if dwpe is None else dwpe.to(dtype), None, None


def embedding(tokens: torch.Tensor, wte: torch.Tensor, wpe: Optional[torch.Tensor] = None, scale: float = 1.0,
              vocab_start: int = 0) -> torch.Tensor:
    return _EmbeddingFn.apply(tokens, wte, wpe, scale, vocab_start)
