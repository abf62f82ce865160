"""Memory-efficient vocabulary output: projection + softmax + NLL loss without materialising the logits.

Capability parity with fairscale/experimental/nn/mevo.py:68-658 (``MemoryEfficientVocabOutput`` with
``tile_factor``, ``reduction``, optional CosFace large-margin cosine loss through ``margin`` / ``scale``, the
``BaselineSoftmax`` / ``BaselineSoftmaxNllLoss`` oracles, ``BackwardTrigger`` so that FSDP finalises a shared
projection weight after the loss's backward).

The reference makes three tiled passes in forward (row max, sum of exponentials, target score), each with its
own recomputation in backward.  Here forward is a single pass with an online softmax (running max and sum per
token, rescaled when the max moves), and backward one recomputation pass that produces ``dX`` and ``dW`` per
tile: a third of the GEMM work forward and half of it backward, with the same peak memory of one
``token_tile x vocab_tile`` block of fp32 logits.
"""

from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn


def _next_power_of_2_or_max(n: int, max_n: int) -> int:
    """Smallest power of two >= n, capped at ``max_n`` (tile sizes)."""
    if n <= 0:
        return 1
    p = 1 << (n - 1).bit_length()
    return min(p, max_n)


def _reshape_inputs(input: torch.Tensor, target: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    if input.dim() == 3:
        input = input.reshape(-1, input.shape[2])
    if target.dim() == 2:
        target = target.reshape(-1)
    return input, target


def get_data(shape: Tuple[Tuple[int, int], Tuple[int, int]], dtype: torch.dtype = torch.float16, device: str = "cuda") -> Tuple[torch.Tensor, nn.Parameter, torch.Tensor]:
    """Random (input, weight, target) of the given ``((tokens, d), (d, vocab))`` shape for tests and benchmarks."""
    (tokens, d1), (d2, vocab) = shape
    assert d1 == d2
    x = torch.rand(tokens, d1, device=device, dtype=dtype).requires_grad_(True)
    w = nn.Parameter(nn.Linear(d2, vocab, bias=False).weight.detach().to(device=device, dtype=dtype))
    t = (torch.rand(tokens, device=device) * vocab).long()
    return x, w, t


class BaselineSoftmax(nn.Module):
    """Un-tiled oracle: full logits, then (log-)softmax in fp32.  ``tile_factor`` is accepted and ignored."""

    def __init__(self, proj_weight: nn.Parameter, tile_factor: int = 0, log_softmax: bool = True, margin: float = 0.35,
                 scale: Optional[float] = None):
        super().__init__()
        self.weight = proj_weight
        self.log_softmax = log_softmax
        self.margin = margin
        self.scale = scale

    def _logits(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        if self.scale is None:
            return F.linear(input, self.weight)
        logits = F.linear(F.normalize(input, dim=1), F.normalize(self.weight, dim=1))
        logits = logits - self.margin * F.one_hot(target, logits.shape[1]).to(logits.dtype)
        return logits * self.scale

    def lmcl_pre_softmax(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        """Large-margin cosine logits: normalised features times normalised class weights, the margin taken off the
        target column, times ``scale``."""
        assert self.scale is not None, "LMCL needs a scale"
        return self._logits(input, target)

    def forward(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        input, target = _reshape_inputs(input, target)
        x = self._logits(input, target)
        return F.log_softmax(x, dim=-1, dtype=torch.float32) if self.log_softmax else F.softmax(x, dim=-1, dtype=torch.float32)


class BaselineSoftmaxNllLoss(BaselineSoftmax):
    def forward(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        input, target = _reshape_inputs(input, target)
        return F.nll_loss(super().forward(input, target), target, reduction="sum")


def lmcl_matmul(i: torch.Tensor, w: torch.Tensor, tgt: torch.Tensor, w_idx: int, margin: float, scale: Optional[float]) -> torch.Tensor:
    """Logits of one vocab tile under LMCL: cosine similarity, margin at the target column, times ``scale``."""
    logits = torch.matmul(F.normalize(i, dim=1), F.normalize(w, dim=1).T)
    cols = torch.arange(w_idx * w.shape[0], (w_idx + 1) * w.shape[0], device=i.device)
    logits = logits - margin * (cols.unsqueeze(0) == tgt.reshape(-1, 1)).to(logits.dtype)
    return logits * scale


class _TiledVocabNll(torch.autograd.Function):
    """sum over tokens of -log softmax(x @ w.T * alpha - margin_at_target * alpha)[target], tile by tile."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w: torch.Tensor, target: torch.Tensor, trigger: Optional[torch.Tensor],  # type: ignore[override]
                tile_t: int, tile_v: int, margin: float, alpha: float) -> torch.Tensor:
        tokens, vocab = x.shape[0], w.shape[0]
        lse = torch.empty(tokens, dtype=torch.float32, device=x.device)
        tgt_logit = torch.empty(tokens, dtype=torch.float32, device=x.device)
        for t0 in range(0, tokens, tile_t):
            xt = x[t0 : t0 + tile_t]
            tt = target[t0 : t0 + tile_t]
            run_max = torch.full((xt.shape[0],), float("-inf"), dtype=torch.float32, device=x.device)
            run_sum = torch.zeros(xt.shape[0], dtype=torch.float32, device=x.device)
            tl = torch.zeros(xt.shape[0], dtype=torch.float32, device=x.device)
            for v0 in range(0, vocab, tile_v):
                logits = _TiledVocabNll._tile_logits(xt, w[v0 : v0 + tile_v], tt, v0, margin, alpha)
                in_tile = (tt >= v0) & (tt < v0 + logits.shape[1])
                idx = (tt - v0).clamp(0, logits.shape[1] - 1)
                tl = torch.where(in_tile, logits.gather(1, idx[:, None]).squeeze(1), tl)
                new_max = torch.maximum(run_max, logits.max(dim=1).values)
                run_sum = run_sum * torch.exp(run_max - new_max) + torch.exp(logits - new_max[:, None]).sum(dim=1)
                run_max = new_max
            lse[t0 : t0 + tile_t] = run_max + torch.log(run_sum)
            tgt_logit[t0 : t0 + tile_t] = tl
        ctx.save_for_backward(x, w, target, lse)
        ctx.cfg = (tile_t, tile_v, margin, alpha, trigger is not None)
        return (lse - tgt_logit).sum()

    @staticmethod
    def _tile_logits(xt: torch.Tensor, wt: torch.Tensor, tt: torch.Tensor, v0: int, margin: float, alpha: float) -> torch.Tensor:
        logits = torch.matmul(xt, wt.T).float()
        if margin != 0.0:
            cols = torch.arange(v0, v0 + wt.shape[0], device=xt.device)
            logits = logits - margin * (cols[None, :] == tt[:, None]).float()
        return logits * alpha if alpha != 1.0 else logits

    @staticmethod
    def backward(ctx: Any, grad_out: torch.Tensor) -> Any:  # type: ignore[override]
        x, w, target, lse = ctx.saved_tensors
        tile_t, tile_v, margin, alpha, has_trigger = ctx.cfg
        dx = torch.zeros_like(x, dtype=torch.float32) if ctx.needs_input_grad[0] else None
        dw = torch.zeros_like(w, dtype=torch.float32) if ctx.needs_input_grad[1] else None
        g = grad_out.float() * alpha
        for t0 in range(0, x.shape[0], tile_t):
            xt, tt = x[t0 : t0 + tile_t], target[t0 : t0 + tile_t]
            for v0 in range(0, w.shape[0], tile_v):
                wt = w[v0 : v0 + tile_v]
                logits = _TiledVocabNll._tile_logits(xt, wt, tt, v0, margin, alpha)
                d = torch.exp(logits - lse[t0 : t0 + tile_t, None])  # softmax probabilities of this tile
                cols = torch.arange(v0, v0 + wt.shape[0], device=x.device)
                d = (d - (cols[None, :] == tt[:, None]).float()) * g
                dl = d.to(x.dtype)
                if dx is not None:
                    dx[t0 : t0 + tile_t] += torch.matmul(dl, wt).float()
                if dw is not None:
                    dw[v0 : v0 + tile_v] += torch.matmul(dl.T, xt).float()
        return (None if dx is None else dx.to(x.dtype), None if dw is None else dw.to(w.dtype), None,
                torch.zeros(1, dtype=w.dtype, device=w.device) if has_trigger else None, None, None, None, None)


def _tile_scores(i: torch.Tensor, w: torch.Tensor, tgt: torch.Tensor, w_idx: int, kernel_obj: Any) -> torch.Tensor:
    """Logits of one vocab tile: plain ``i @ w.T``, or the LMCL form while the module has a ``scale``."""
    if kernel_obj.scale is None:
        return torch.matmul(i, w.T)
    return lmcl_matmul(i, w, tgt, w_idx, kernel_obj.margin, kernel_obj.scale)


def _target_scores(i: torch.Tensor, w: torch.Tensor, target: torch.Tensor, kernel_obj: Any) -> torch.Tensor:
    if kernel_obj.scale is None:
        return (i.float() * w.float()[target]).sum(dim=1)
    cos = (F.normalize(i.float(), dim=1) * F.normalize(w.float(), dim=1)[target]).sum(dim=1)
    return kernel_obj.scale * (cos - kernel_obj.margin)


class GetMaxFunction(torch.autograd.Function):
    """Row maximum of ``i @ w.T`` (no gradient): the first of the three passes of the reference's formulation
    (fairscale/experimental/nn/mevo.py:201-263).  ``MemoryEfficientVocabOutput`` here needs a single pass
    (:class:`_TiledVocabNll`); the three functions remain for code that composes the loss itself."""

    @staticmethod
    def forward(ctx: Any, i: torch.Tensor, w: torch.Tensor, tgt: torch.Tensor, kernel_obj: Any, w_idx: int = 0) -> torch.Tensor:  # type: ignore[override]
        return _tile_scores(i, w, tgt, w_idx, kernel_obj).float().max(dim=1).values

    @staticmethod
    def backward(ctx: Any, *grad: Any) -> Any:  # type: ignore[override]
        return None, None, None, None, None  # the maximum only stabilises the exponentials: it carries no gradient


class GetSumFunction(torch.autograd.Function):
    """``sum_v exp(logit_v - maxs)`` per token, with the gradient recomputed from ``i`` and ``w`` in backward instead of
    keeping the ``[tokens, vocab]`` logits (parity: fairscale/experimental/nn/mevo.py:266-354)."""

    @staticmethod
    def forward(ctx: Any, i: torch.Tensor, w: torch.Tensor, tgt: torch.Tensor, maxs: torch.Tensor, kernel_obj: Any, w_idx: int = 0) -> torch.Tensor:  # type: ignore[override]
        ctx.save_for_backward(i, w, tgt, maxs)
        ctx.kernel_obj, ctx.w_idx = kernel_obj, w_idx
        logits = _tile_scores(i, w, tgt, w_idx, kernel_obj).float()
        return (logits - maxs.reshape(-1, 1)).exp().sum(dim=1)

    @staticmethod
    def backward(ctx: Any, *grad: Any) -> Any:  # type: ignore[override]
        i, w, tgt, maxs = ctx.saved_tensors
        with torch.enable_grad():
            i2, w2 = i.detach().requires_grad_(), w.detach().requires_grad_()
            logits = _tile_scores(i2, w2, tgt, ctx.w_idx, ctx.kernel_obj).float()
            out = (logits - maxs.reshape(-1, 1)).exp().sum(dim=1)
            gi, gw = torch.autograd.grad(out, (i2, w2), grad[0])
        return gi, gw, None, None, None, None


class TargetScoreFunction(torch.autograd.Function):
    """Logit of each token's target class, ``(i * w[target]).sum(1)`` with the LMCL margin / scale applied
    (parity: fairscale/experimental/nn/mevo.py:357-445)."""

    @staticmethod
    def forward(ctx: Any, i: torch.Tensor, w: torch.Tensor, target: torch.Tensor, kernel_obj: Any) -> torch.Tensor:  # type: ignore[override]
        ctx.save_for_backward(i, w, target)
        ctx.kernel_obj = kernel_obj
        return _target_scores(i, w, target, kernel_obj)

    @staticmethod
    def backward(ctx: Any, *grad: Any) -> Any:  # type: ignore[override]
        i, w, target = ctx.saved_tensors
        with torch.enable_grad():
            i2, w2 = i.detach().requires_grad_(), w.detach().requires_grad_()
            gi, gw = torch.autograd.grad(_target_scores(i2, w2, target, ctx.kernel_obj), (i2, w2), grad[0].float())
        return gi, gw, None, None


class BackwardTriggerFn(torch.autograd.Function):
    """Pass the weight through and tie a tiny trigger parameter into the graph (it receives a zero gradient)."""

    @staticmethod
    def forward(ctx: Any, w: torch.Tensor, trigger_tensor: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        ctx.save_for_backward(trigger_tensor)
        return w.view_as(w)

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor) -> Any:  # type: ignore[override]
        (trigger,) = ctx.saved_tensors
        return grad, torch.zeros_like(trigger)


class BackwardTrigger(nn.Module):
    """Owns a 1-element parameter whose ``_linked_param`` is the (shared) weight; a sharded data-parallel wrapper
    that sees this parameter's gradient hook fire knows the linked weight's gradient is complete."""

    def __init__(self, linked_param: torch.Tensor):
        super().__init__()
        assert isinstance(linked_param, nn.Parameter)
        self.trigger = nn.Parameter(torch.rand(1, dtype=linked_param.dtype, device=linked_param.device))
        self.trigger._linked_param = linked_param  # type: ignore[attr-defined]

    def forward(self) -> torch.Tensor:  # type: ignore[override]
        return BackwardTriggerFn.apply(self.trigger._linked_param, self.trigger)


class MemoryEfficientVocabOutput(nn.Module):
    """Args:
        proj_weight: ``[vocab, d_model]`` weight, usually shared with the token embedding.
        tile_factor: number of splits of the token and of the vocab dimension (default 16).
        reduction: ``"sum"`` or ``"mean"`` over tokens.
        margin, scale: LMCL hyper-parameters; LMCL is off while ``scale`` is None.
    """

    def __init__(self, proj_weight: nn.Parameter, tile_factor: int = 16, reduction: str = "sum", margin: float = 0.35,
                 scale: Optional[float] = None):
        super().__init__()
        assert reduction in ["sum", "mean"]
        self.proj_weight = proj_weight
        self.tf_in, self.tf_w = tile_factor, tile_factor
        self.log_softmax = True
        self.reduction = reduction
        self.margin = margin
        self.scale = scale
        self.trigger = BackwardTrigger(self.proj_weight)

    def get_target_nlprob(self, i: torch.Tensor, w: torch.Tensor, target: torch.Tensor, debase_max: torch.Tensor,
                          exp_sums: torch.Tensor) -> torch.Tensor:
        """Summed negative log-probability of the targets from already known softmax statistics: ``debase_max`` is the
        row maximum of the logits and ``exp_sums`` the row sum of ``exp(logit - max)`` (parity:
        fairscale/experimental/nn/mevo.py:576-586; the single-pass loss above does not need it)."""
        prob = (_target_scores(i, w, target, self) - debase_max).exp() / exp_sums
        if self.log_softmax:
            prob = prob.log()
        return -prob.sum()

    def eval_forward(self, input: torch.Tensor) -> torch.Tensor:
        """Plain logits (no target given at evaluation time)."""
        return torch.matmul(input, self.proj_weight.T)

    def forward(self, input: torch.Tensor, target: Optional[torch.Tensor]) -> torch.Tensor:  # type: ignore[override]
        if not self.training and target is None:
            return self.eval_forward(input)
        assert isinstance(input, torch.Tensor) and isinstance(target, torch.Tensor)
        if torch.is_grad_enabled():
            assert input.requires_grad
        input, target = _reshape_inputs(input, target)
        tokens, d_model = input.shape
        vocab, d2 = self.proj_weight.shape
        assert d_model == d2, f"incorrect shape {d_model} vs {d2}"
        assert target.shape == (tokens,), f"incorrect shape {tokens} vs {tuple(target.shape)}"
        tile_t = _next_power_of_2_or_max(tokens // self.tf_in, tokens)
        tile_v = _next_power_of_2_or_max(vocab // self.tf_w, vocab)
        w = self.proj_weight
        if self.scale is not None:  # cosine logits: normalisation stays in autograd, tiles work on unit vectors
            x_in, w_in, margin, alpha = F.normalize(input, dim=1), F.normalize(w, dim=1), self.margin, float(self.scale)
        else:
            x_in, w_in, margin, alpha = input, w, 0.0, 1.0
        loss = _TiledVocabNll.apply(x_in, w_in, target, self.trigger.trigger, tile_t, tile_v, margin, alpha)
        return loss / tokens if self.reduction == "mean" else loss
