"""Cross entropy over vocabulary-sharded logits.

Parity: fairscale/nn/model_parallel/cross_entropy.py:29-106 (per-token loss, no reduction).  The reference
issues three all-reduces (max, target logit, sum-exp) around a chain of ATen ops and keeps a full softmax
for backward.  Here every rank computes the triple ``(max, sum-exp at that max, target logit)`` per token in
one pass over its logits shard, the triples are combined with ONE all-gather of 3 floats per token, and
backward regenerates the softmax from the saved log-sum-exp in one pass (no saved softmax).
"""

from __future__ import annotations

from typing import Any

import torch

from ...ops.loss import ce_backward, ce_forward
from ...parallel import comm
from .initialize import get_model_parallel_group, get_model_parallel_rank, get_model_parallel_world_size
from .utils import VocabUtility


__all__ = [
    "vocab_parallel_cross_entropy",
]


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, vocab_parallel_logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        group = get_model_parallel_group()
        world = get_model_parallel_world_size()
        rank = get_model_parallel_rank()
        V = vocab_parallel_logits.size(-1)
        v0, _ = VocabUtility.vocab_range_from_per_partition_vocab_size(V, rank, world)
        logits2d = vocab_parallel_logits.reshape(-1, V)
        tgt = target.reshape(-1)
        _, _, stats = ce_forward(logits2d, tgt, ignore_index=-(2**62), vocab_start=v0, want_stats=True)
        assert stats is not None
        if world > 1:
            gathered = torch.empty((world,) + tuple(stats.shape), dtype=stats.dtype, device=stats.device)
            comm.all_gather_into(gathered.view(-1), stats.contiguous().view(-1), group=group)
        else:
            gathered = stats.unsqueeze(0)
        gmax = gathered[..., 0].max(dim=0).values
        sumexp = (gathered[..., 1] * torch.exp(gathered[..., 0] - gmax)).sum(dim=0)
        target_logit = gathered[..., 2].sum(dim=0)
        lse = gmax + torch.log(sumexp)
        loss = (lse - target_logit).view_as(target)
        ctx.save_for_backward(logits2d, tgt, lse)
        ctx.v0 = v0
        ctx.shape = vocab_parallel_logits.shape
        return loss.to(torch.float32)

    @staticmethod
    def backward(ctx: Any, grad_output: torch.Tensor):  # type: ignore[override]
        logits2d, tgt, lse = ctx.saved_tensors
        g = grad_output.reshape(-1).float().contiguous()
        # the loss is the last consumer of the logits, so their storage is reused for the gradient
        grad = ce_backward(logits2d, tgt, lse, g, 1.0, ignore_index=-(2**62), vocab_start=ctx.v0, inplace=logits2d.is_cuda)
        return grad.view(ctx.shape), None


def vocab_parallel_cross_entropy(vocab_parallel_logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Per-token cross entropy for logits whose last dimension is this rank's vocabulary shard."""
    return _VocabParallelCrossEntropy.apply(vocab_parallel_logits, target)
