"""Top-2 gating (GShard) in index form.

Behavioural parity with fairscale/nn/moe/top2gate.py:37-130: fp32 softmax, top-1 by probability, second
expert by Gumbel-max on the logits with the first masked out, slot assignment by token order with the second
choices queued behind all first choices, capacity ``2*S/E``, auxiliary loss ``mean(me * ce)``, gates
renormalised over the kept experts.

The reference materialises one-hot ``[S, E, C]`` tensors (537 MB fp32 for S=8192, E=64, C=256) and dispatches
with dense einsums.  Here routing is kept as per-token ``(expert, slot, gate)`` triples (:class:`Top2Route`);
the dense ``(l_aux, combine_weights, dispatch_mask)`` contract is still available from :func:`top2gating` for
code that wants it and is what ``Top2Gate.forward`` returns.
"""

from __future__ import annotations

from typing import Callable, Dict, NamedTuple, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

gumbel_map: Dict[torch.device, Callable] = {}


def gumbel_rsample(shape: Tuple, device: torch.device) -> Tensor:
    sampler = gumbel_map.get(device)
    if sampler is None:
        one = torch.tensor(1.0, device=device)
        zero = torch.tensor(0.0, device=device)
        sampler = torch.distributions.gumbel.Gumbel(zero, one).rsample  # type: ignore[assignment]
        gumbel_map[device] = sampler
    return sampler(shape)


def one_hot(tensor: torch.Tensor, num_classes: int) -> Tensor:
    assert num_classes > 0, "num_classes must be a positive integer"
    ret = torch.zeros(tensor.shape + (num_classes,), device=tensor.device, dtype=tensor.dtype)
    ret.scatter_(-1, tensor.unsqueeze(-1), 1)
    return ret


class Top2Route(NamedTuple):
    """Routing of ``S`` tokens to ``E`` experts with ``capacity`` slots each.

    ``expert[s, k]`` / ``slot[s, k]``: k-th choice of token s and its position in that expert's buffer;
    ``keep[s, k]``: False when the choice overflowed the capacity; ``gate[s, k]``: normalised weight (0 if
    dropped, differentiable w.r.t. the logits); ``l_aux``: load-balancing loss.
    """

    l_aux: Tensor
    expert: Tensor
    slot: Tensor
    keep: Tensor
    gate: Tensor
    capacity: int
    num_experts: int
    counts: Optional[Tensor] = None  # int32 [2 * E]: tokens per expert as first / second choice (CUDA index kernels only)


def _route_indices_native(logits: Tensor, noise: Tensor) -> Optional[Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]]:
    """(idx1, idx2, loc1, loc2, count1) from the three-launch CUDA path, or None when it does not apply."""
    from ...ops import _bind

    S, E = logits.shape
    if not (_bind.use_native(logits) and logits.dtype in (torch.float32, torch.bfloat16) and 2 <= E <= 512 and logits.is_contiguous()):
        return None
    from ctypes import c_int, c_void_p

    _bind._SIGNATURES.setdefault("fsb_top2_workspace_ints", [c_int, c_int])
    _bind._SIGNATURES.setdefault("fsb_top2_route", [c_void_p, c_int, c_void_p, c_int, c_int] + [c_void_p] * 7)
    dev = logits.device
    out = torch.empty((4, S), dtype=torch.int32, device=dev)
    ws = torch.empty(_bind.fn("fsb_top2_workspace_ints")(S, E), dtype=torch.int32, device=dev)
    totals = torch.empty(2 * E, dtype=torch.int32, device=dev)
    noise = noise.to(torch.float32).contiguous()
    _bind.call("fsb_top2_route", logits.data_ptr(), _bind.dtype_code(logits.dtype), noise.data_ptr(), S, E, out[0].data_ptr(),
               out[1].data_ptr(), out[2].data_ptr(), out[3].data_ptr(), ws.data_ptr(), totals.data_ptr(), _bind.stream_ptr(dev), launches=3)
    return out, totals


class _GateValues(torch.autograd.Function):
    """Softmax, the two kept gate values (renormalised) and the auxiliary loss in one kernel, with a one-kernel backward
    (``csrc/top2gate.cu``).  ``route`` is the int32 ``[4, S]`` output of the index kernels (idx1, idx2, loc1, loc2)."""

    @staticmethod
    def forward(ctx, logits: Tensor, route: Tensor, count1: Tensor, capacity: int):  # type: ignore[override]
        from ctypes import c_float, c_int, c_void_p

        from ...ops import _bind

        _bind._SIGNATURES.setdefault("fsb_top2_gate_fwd", [c_void_p, c_int, c_int, c_int] + [c_void_p] * 4 + [c_int, c_float] + [c_void_p] * 6)
        S, E = logits.shape
        dev = logits.device
        gate = torch.empty((S, 2), dtype=torch.float32, device=dev)
        scratch = torch.zeros(E + 2, dtype=torch.float32, device=dev)  # column sums | l_aux | ticket
        eps = float(torch.finfo(torch.float32).eps)
        _bind.call("fsb_top2_gate_fwd", logits.data_ptr(), _bind.dtype_code(logits.dtype), S, E, route[0].data_ptr(), route[1].data_ptr(),
                   route[2].data_ptr(), route[3].data_ptr(), capacity, eps, count1.data_ptr(), gate.data_ptr(), scratch.data_ptr(),
                   scratch[E:].data_ptr(), scratch[E + 1:].data_ptr(), _bind.stream_ptr(dev))
        ctx.save_for_backward(logits, route, count1)
        ctx.capacity, ctx.eps = capacity, eps
        return gate, scratch[E]

    @staticmethod
    def backward(ctx, d_gate: Tensor, d_l_aux: Tensor):  # type: ignore[override]
        from ctypes import c_float, c_int, c_void_p

        from ...ops import _bind

        _bind._SIGNATURES.setdefault("fsb_top2_gate_bwd", [c_void_p, c_int, c_int, c_int] + [c_void_p] * 4 + [c_int, c_float] + [c_void_p] * 5)
        logits, route, count1 = ctx.saved_tensors
        S, E = logits.shape
        d_logits = torch.empty_like(logits)
        d_gate = d_gate.to(torch.float32).contiguous()
        d_aux = d_l_aux.to(torch.float32).reshape(1).contiguous()
        _bind.call("fsb_top2_gate_bwd", logits.data_ptr(), _bind.dtype_code(logits.dtype), S, E, route[0].data_ptr(), route[1].data_ptr(),
                   route[2].data_ptr(), route[3].data_ptr(), ctx.capacity, ctx.eps, d_gate.data_ptr(), d_aux.data_ptr(), count1.data_ptr(),
                   d_logits.data_ptr(), _bind.stream_ptr(logits.device))
        return d_logits, None, None, None


def top2_route(logits: torch.Tensor, noise: Optional[Tensor] = None) -> Top2Route:
    """Index-form top-2 routing; ``noise`` (Gumbel, same shape as ``logits``) can be supplied for reproducibility.

    On CUDA everything runs in the kernels of ``csrc/top2gate.cu``: three launches for the index part (two arg-maxes, slot
    assignment in token order, per-expert counts) and one for the differentiable part (fp32 softmax, renormalised gate
    values, auxiliary loss), whose backward is one more kernel.  The eager formulation below is the CPU path and the
    oracle of the kernels' tests."""
    S, E = logits.shape
    capacity = 2 * S // E
    assert S % E == 0
    if noise is None:
        noise = gumbel_rsample(logits.shape, device=logits.device)
    if logits.is_cuda and not logits.is_contiguous():
        logits = logits.contiguous()
    native = _route_indices_native(logits.detach(), noise) if logits.is_cuda else None
    if native is not None:
        # five launches in all: three for the indices, one for softmax + gate values + auxiliary loss, one memset
        route, counts2 = native
        count1 = counts2[:E]
        gate, l_aux = _GateValues.apply(logits, route, count1, capacity)
        r = route.long()
        keep = torch.stack([r[2] < capacity, r[3] < capacity], dim=1)
        expert = torch.stack([r[0], r[1]], dim=1)
        slot = torch.stack([r[2], r[3]], dim=1) * keep
        return Top2Route(l_aux.to(logits.dtype), expert, slot, keep, gate, capacity, E, counts2)
    gates = F.softmax(logits, dim=1, dtype=torch.float)
    idx1 = torch.argmax(gates, dim=1)
    noisy = (logits + noise).scatter(1, idx1.unsqueeze(1), float("-inf"))
    idx2 = torch.argmax(noisy, dim=1)
    mask1 = one_hot(idx1, E)
    mask2 = one_hot(idx2, E)
    # position of each token among the tokens that chose the same expert, in token order
    loc1 = (torch.cumsum(mask1, dim=0) - 1).gather(1, idx1.unsqueeze(1)).squeeze(1)
    loc2 = (torch.cumsum(mask2, dim=0) - 1 + mask1.sum(dim=0, keepdim=True)).gather(1, idx2.unsqueeze(1)).squeeze(1)
    ce = mask1.float().mean(dim=0)

    me = gates.mean(dim=0)
    l_aux = torch.mean(me * ce)

    keep1, keep2 = loc1 < capacity, loc2 < capacity
    g1 = gates.gather(1, idx1.unsqueeze(1)).squeeze(1) * keep1
    g2 = gates.gather(1, idx2.unsqueeze(1)).squeeze(1) * keep2
    denom = torch.clamp(g1 + g2, min=torch.finfo(g1.dtype).eps)
    gate = torch.stack([g1 / denom, g2 / denom], dim=1)
    expert = torch.stack([idx1, idx2], dim=1)
    slot = torch.stack([loc1 * keep1, loc2 * keep2], dim=1)
    keep = torch.stack([keep1, keep2], dim=1)
    return Top2Route(l_aux.to(logits.dtype), expert, slot, keep, gate, capacity, E)


def dense_from_route(route: Top2Route, dtype: torch.dtype) -> Tuple[Tensor, Tensor]:
    """``combine_weights [S, E, C]`` and ``dispatch_mask [S, E, C]`` (bool) from index-form routing."""
    S = route.expert.shape[0]
    combine = torch.zeros((S, route.num_experts, route.capacity), dtype=route.gate.dtype, device=route.gate.device)
    rows = torch.arange(S, device=route.expert.device)
    for k in range(2):
        w = route.gate[:, k] * route.keep[:, k]
        combine = combine.index_put((rows, route.expert[:, k], route.slot[:, k]), w, accumulate=True)
    return combine.to(dtype), combine.bool()


def top2gating(logits: torch.Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    """Dense Top-2 gating: ``(l_aux, combine_weights[S,E,C], dispatch_mask[S,E,C])``."""
    route = top2_route(logits)
    combine, mask = dense_from_route(route, logits.dtype)
    return route.l_aux, combine, mask


class _GateProjection(torch.autograd.Function):
    """``logits[T, E] = x[T, d] @ wg[E, d]^T`` in fp32 for bf16 activations on the GPU: the product runs on the tcgen05 GEMM
    (bf16 operands, fp32 accumulation and fp32 output) with the expert dimension zero-padded to one 128-row tile."""

    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor) -> Tensor:  # type: ignore[override]
        from ...ops import gemm as gemm_ops

        E, d = w.shape
        x2 = x.reshape(-1, d)
        w_pad = torch.zeros((-(-E // 128) * 128, d), dtype=torch.bfloat16, device=x.device)
        w_pad[:E].copy_(w)
        logits, _ = gemm_ops.linear_forward(x2, w_pad, None, out_dtype=torch.float32)
        ctx.save_for_backward(x2, w_pad)
        ctx.meta = (E, x.shape, w.dtype)
        # contiguous: the routing kernels take dense [S, E] logits (a strided slice would send them down the eager path)
        return logits[:, :E].contiguous().reshape(*x.shape[:-1], E)

    @staticmethod
    def backward(ctx, d_logits: Tensor):  # type: ignore[override]
        from ...ops import gemm as gemm_ops

        x2, w_pad = ctx.saved_tensors
        E, x_shape, w_dtype = ctx.meta
        dl = torch.zeros((x2.shape[0], w_pad.shape[0]), dtype=torch.bfloat16, device=x2.device)
        dl[:, :E].copy_(d_logits.reshape(-1, E))
        dx = gemm_ops.linear_dgrad(dl, w_pad).view(x_shape) if ctx.needs_input_grad[0] else None
        dw = gemm_ops.linear_wgrad(dl, x2)[:E].to(w_dtype) if ctx.needs_input_grad[1] else None
        return dx, dw


def gate_logits(x: Tensor, wg: torch.nn.Linear) -> Tensor:
    """Router logits in fp32 (the softmax over experts is taken in fp32 whatever the activations' dtype)."""
    w = wg.weight
    if x.is_cuda and x.dtype == torch.bfloat16 and w.shape[1] % 8 == 0:
        from ...ops import _bind

        if _bind.use_native(x):
            return _GateProjection.apply(x, w)
    if x.dtype != w.dtype:
        return torch.nn.functional.linear(x.float(), w.float())
    return wg(x)


class Top2Gate(torch.nn.Module):
    """Gate network ``wg: model_dim -> num_experts`` followed by top-2 routing.

    ``forward`` returns the dense triple of the reference; :meth:`route` returns the index form that
    :class:`~fairscale_b200.nn.moe.MOELayer` uses for its scatter / gather fast path.
    """

    wg: torch.nn.Linear

    def __init__(self, model_dim: int, num_experts: int) -> None:
        super().__init__()
        self.wg = torch.nn.Linear(model_dim, num_experts, bias=False)

    def route(self, input: torch.Tensor) -> Top2Route:
        return top2_route(gate_logits(input, self.wg))

    def forward(self, input: torch.Tensor) -> Tuple[Tensor, Tensor, Tensor]:  # type: ignore[override]
        return top2gating(gate_logits(input, self.wg))
