"""Softmax cross-entropy on bf16 logits (``csrc/cross_entropy.cu``)."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _bind


def ce_forward(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100, vocab_start: int = 0,
               want_stats: bool = False) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Per-row loss and log-sum-exp of ``logits[rows, V]``; optional ``(max, sumexp, target_logit)`` stats."""
    rows, V = logits.shape
    if not _bind.use_native(logits) or logits.dtype != torch.bfloat16 or logits.stride(0) % 8:
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1)
        local = targets - vocab_start
        inside = (local >= 0) & (local < V) & (targets != ignore_index)
        tl = torch.where(inside, lf.gather(1, local.clamp(0, V - 1).unsqueeze(1)).squeeze(1), torch.zeros_like(lse))
        loss = torch.where(targets == ignore_index, torch.zeros_like(lse), lse - tl)
        stats = None
        if want_stats:
            m = lf.max(dim=-1).values
            stats = torch.stack([m, torch.exp(lf - m.unsqueeze(1)).sum(-1), tl], dim=1)
        return loss, lse, stats
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    stats = torch.empty((rows, 3), dtype=torch.float32, device=logits.device) if want_stats else None
    _bind.call("fsb_ce_fwd", logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), lse.data_ptr(), _bind.ptr(stats), rows, V,
               logits.stride(0), vocab_start, ignore_index, _bind.stream_ptr(logits.device))
    return loss, lse, stats


def ce_backward(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, grad_out: torch.Tensor, scale: float,
                ignore_index: int = -100, vocab_start: int = 0, inplace: bool = True) -> torch.Tensor:
    """``(softmax - onehot) * grad_out * scale``; overwrites ``logits`` when ``inplace``."""
    rows, V = logits.shape
    if not _bind.use_native(logits) or logits.dtype != torch.bfloat16 or logits.stride(0) % 8:
        p = torch.exp(logits.float() - lse.unsqueeze(1))
        local = targets - vocab_start
        inside = (local >= 0) & (local < V)
        onehot = torch.zeros_like(p)
        onehot[inside, local[inside]] = 1.0
        g = grad_out.float().reshape(-1) * scale
        g = g.expand(rows) if g.numel() == 1 else g
        g = torch.where(targets == ignore_index, torch.zeros_like(g), g)
        return ((p - onehot) * g.unsqueeze(1)).to(logits.dtype)
    out = logits if inplace else torch.empty_like(logits)
    g = grad_out.float().contiguous()
    _bind.call("fsb_ce_bwd", logits.data_ptr(), targets.data_ptr(), lse.data_ptr(), g.data_ptr(), int(g.numel() == 1), scale,
               out.data_ptr(), rows, V, logits.stride(0), vocab_start, ignore_index, _bind.stream_ptr(logits.device))
    return out


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ignore_index: int):  # type: ignore[override]
        l2 = logits.reshape(-1, logits.shape[-1])
        t = targets.reshape(-1)
        loss, lse, _ = ce_forward(l2, t, ignore_index)
        valid = (t != ignore_index).sum().clamp(min=1).float() if ignore_index >= 0 else None
        ctx.save_for_backward(l2, t, lse, valid)
        ctx.ignore_index = ignore_index
        ctx.shape = logits.shape
        total = loss.sum()
        return total / (valid if valid is not None else float(t.numel()))

    @staticmethod
    def backward(ctx, grad_out):  # type: ignore[override]
        l2, t, lse, valid = ctx.saved_tensors
        if valid is not None:
            g = grad_out / valid
            scale = 1.0
        else:
            g = grad_out
            scale = 1.0 / t.numel()
        # the logits are dead after this point (the loss is the last consumer), so they are reused for the gradient
        dl = ce_backward(l2, t, lse, g.reshape(1), scale, ctx.ignore_index, inplace=True)
        return dl.view(ctx.shape), None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean token cross-entropy.  NOTE: the backward pass overwrites ``logits`` with its gradient."""
    return _CrossEntropyFn.apply(logits, targets, ignore_index)
