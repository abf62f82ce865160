"""Mixture-of-experts layer with expert parallelism.

API parity with fairscale/nn/moe/moe_layer.py:23-91 (``MOELayer(gate, experts, group)``, ``l_aux``, expert
parameters tagged ``p.expert = True``, the ``(l_aux, combine_weights, dispatch_mask)`` gate contract).

Two data paths:

* **index path** (gates exposing ``route()``, e.g. :class:`Top2Gate`): tokens are scattered to
  ``(expert, slot)`` rows and gathered back with their gate weights; no ``[S, E, C]`` tensor exists.  With an
  NVLink workspace for the group the scatter writes rows *directly into the destination rank's expert buffer*
  and the combine reads rows directly from the owners' output buffers (``csrc/comm.cu``), fusing dispatch /
  combine with the all-to-all; otherwise a local scatter + ``all_to_all_single`` is used (NCCL / gloo).
* **dense path** (any other gate): the reference's einsum formulation.
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Any, Optional, Tuple, Union, cast

import torch
import torch.distributed as dist
from torch import Tensor
from torch.nn import Module, ModuleList

from ...parallel import comm, symm
from .top2gate import Top2Route

if TYPE_CHECKING:
    Base = Module[Tensor]
else:
    Base = Module


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, group: Any, input: Tensor) -> Tensor:  # type: ignore[override]
        ctx.group = group
        input = input.contiguous()
        output = torch.empty_like(input)
        comm.all_to_all_single(output, input, group)
        return output

    @staticmethod
    def backward(ctx: Any, *grad_output: Tensor) -> Tuple[None, Tensor]:  # type: ignore[override]
        return (None, _AllToAll.apply(ctx.group, *grad_output))


class _LayerBuffers:
    """The symmetric-heap buffers of one MOELayer (landing buffer of the dispatch, expert outputs for the combine, and the
    combine's gradient landing buffer).  A layer that uses its own buffers needs no defensive copies: what the dispatch
    lands is read in place by the experts and kept for their backward, the expert outputs stay where the backward reads them
    again.  That holds while at most one forward of the layer is waiting for its backward; a second forward in between
    (micro-batches run forward first, backward later) falls back to shared buffers plus copies."""

    _count = 0  # construction order is the same on every rank

    def __init__(self) -> None:
        self.index = _LayerBuffers._count
        _LayerBuffers._count += 1
        self.outstanding = 0
        self.full = False
        self.expect_backward = False

    def _allocate(self, ws: Any, rows: int, M: int, dtype: torch.dtype) -> bool:
        if self.full:
            return False
        try:
            self.bufs = {w: ws.scratch(f"moe{self.index}:{w}", (rows, M), dtype) for w in ("in", "out", "grad")}
            return True
        except MemoryError:
            self.full = True  # the heap has no room for per-layer buffers (the same on every rank): shared buffers + copies
            return False

    def claim(self, ws: Any, rows: int, M: int, dtype: torch.dtype) -> bool:
        """Called by a dispatch forward: True if this forward may use the layer's own buffers (``self.bufs``).
        ``self.expect_backward`` is set by the layer before the call (grad mode is off inside ``Function.forward``)."""
        self._mine = False
        if self.outstanding > 0 or not self._allocate(ws, rows, M, dtype):
            return False
        if self.expect_backward:
            self.outstanding += 1  # released by the dispatch's backward
        self._mine = True
        return True

    def holds(self) -> bool:
        """For the combine of the same forward: did its dispatch get the layer's own buffers?"""
        return bool(getattr(self, "_mine", False))

    def release(self) -> None:
        if self.outstanding > 0:
            self.outstanding -= 1


def _routes(route: Top2Route, world: int, n_local: int, rank: int) -> Tuple[Tensor, Tensor, Tensor]:
    """Per (token, choice): destination rank (-1 if dropped), row in the destination's
    ``[n_local, world * C, M]`` buffer, and flat slot ``expert * C + slot`` in the global ``[E, C, M]`` view."""
    C = route.capacity
    e = route.expert
    dst_rank = torch.where(route.keep, e // n_local, torch.full_like(e, -1))
    dst_row = (e % n_local) * (world * C) + rank * C + route.slot
    flat = e * C + route.slot
    return dst_rank.to(torch.int32).contiguous(), dst_row.to(torch.int32).contiguous(), flat


class _Dispatch(torch.autograd.Function):
    """tokens ``[S, M]`` -> expert inputs ``[n_local, world * C, M]`` on the owning ranks."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, route: Top2Route, group: Any, n_local: int, owner: Optional[_LayerBuffers] = None) -> Tensor:  # type: ignore[override]
        world, rank = comm.group_size(group), comm.group_rank(group)
        C, E, M = route.capacity, route.num_experts, x.shape[1]
        dst_rank, dst_row, flat = _routes(route, world, n_local, rank)
        ctx.meta = (group, n_local, world, rank, C, E, M, x.dtype)
        ctx.owner, ctx.claimed = owner, False
        ctx.save_for_backward(dst_rank, dst_row, flat, route.keep)
        ws = symm.workspace_for(group) if (x.is_cuda and comm.comm_mode() == "fused" and x.dtype == torch.bfloat16) else None
        if owner is not None:
            owner._mine = False
        if ws is not None:
            private = owner is not None and owner.claim(ws, n_local * world * C, M, x.dtype)
            ctx.claimed = private and owner.expect_backward
            buf = owner.bufs["in"] if private else ws.scratch("moe_in", (n_local * world * C, M), x.dtype)
            fill = (route.counts, E, C, n_local) if route.counts is not None else None
            if fill is None:
                buf.zero_()  # without per-expert counts the kernel cannot tell which rows stay unclaimed
            ws.moe_scatter_rows(buf, x.contiguous(), dst_rank.view(-1), dst_row.view(-1), None, 2, fill=fill)
            out = buf.view(n_local, world * C, M)
            # the layer's own landing buffer stays untouched until its backward: the experts read it in place
            return out if private else out.clone()
        local = x.new_zeros((E * C, M))
        for k in range(2):
            kept = route.keep[:, k]
            local.index_copy_(0, flat[kept, k], x[kept])
        out = torch.empty_like(local)
        comm.all_to_all_single(out, local, group)  # [world, n_local, C, M] by source rank
        return out.view(world, n_local, C, M).transpose(0, 1).reshape(n_local, world * C, M)

    @staticmethod
    def backward(ctx: Any, grad: Tensor):  # type: ignore[override]
        group, n_local, world, rank, C, E, M, dtype = ctx.meta
        dst_rank, dst_row, flat, keep = ctx.saved_tensors
        S = dst_rank.shape[0]
        if ctx.claimed:
            ctx.owner.release()
        ws = symm.workspace_for(group) if (grad.is_cuda and comm.comm_mode() == "fused" and grad.dtype == torch.bfloat16) else None
        if ws is not None:
            buf = ws.scratch("moe_dgrad", (n_local * world * C, M), grad.dtype)
            buf.copy_(grad.reshape(-1, M))
            dx = torch.empty((S, M), dtype=grad.dtype, device=grad.device)
            ws.moe_gather_rows(buf, dx, dst_rank.view(-1), dst_row.view(-1), None, 2)
            return dx, None, None, None, None
        g = grad.view(n_local, world, C, M).transpose(0, 1).contiguous().view(E * C, M)
        back = torch.empty_like(g)
        comm.all_to_all_single(back, g, group)
        dx = grad.new_zeros((S, M))
        for k in range(2):
            kept = keep[:, k]
            dx[kept] += back[flat[kept, k]]
        return dx, None, None, None, None


class _Combine(torch.autograd.Function):
    """expert outputs ``[n_local, world * C, M]`` -> tokens ``[S, M]`` weighted by the gates."""

    @staticmethod
    def forward(ctx: Any, expert_out: Tensor, gate: Tensor, route: Top2Route, group: Any, n_local: int,
                owner: Optional[_LayerBuffers] = None) -> Tensor:  # type: ignore[override]
        world, rank = comm.group_size(group), comm.group_rank(group)
        C, E, M = route.capacity, route.num_experts, expert_out.shape[-1]
        dst_rank, dst_row, flat = _routes(route, world, n_local, rank)
        S = dst_rank.shape[0]
        w = (gate * route.keep).to(torch.float32).contiguous()
        ctx.meta = (group, n_local, world, rank, C, E, M)
        ctx.fill = (route.counts, E, C, n_local) if route.counts is not None else None
        ws = symm.workspace_for(group) if (expert_out.is_cuda and comm.comm_mode() == "fused" and expert_out.dtype == torch.bfloat16) else None
        ctx.private = ws is not None and owner is not None and owner.holds()
        ctx.owner = owner
        if ws is not None:
            buf = owner.bufs["out"] if ctx.private else ws.scratch("moe_out", (n_local * world * C, M), expert_out.dtype)
            buf.copy_(expert_out.reshape(-1, M))
            out = torch.empty((S, M), dtype=expert_out.dtype, device=expert_out.device)
            ws.moe_gather_rows(buf, out, dst_rank.view(-1), dst_row.view(-1), w.view(-1), 2)
            # the layer's own buffer keeps the expert outputs until the backward reads them remotely again
            ctx.save_for_backward(dst_rank, dst_row, flat, route.keep, w, buf if ctx.private else expert_out)
            return out
        eo = expert_out.view(n_local, world, C, M).transpose(0, 1).contiguous().view(E * C, M)
        home = torch.empty_like(eo)
        comm.all_to_all_single(home, eo, group)  # rows of the global [E, C, M] view that came from this rank's tokens
        rows = torch.stack([home[flat[:, 0]], home[flat[:, 1]]], dim=1)  # [S, 2, M]
        out = (rows.float() * w.unsqueeze(-1)).sum(dim=1).to(expert_out.dtype)
        ctx.save_for_backward(dst_rank, dst_row, flat, route.keep, w, rows)
        return out

    @staticmethod
    def backward(ctx: Any, dy: Tensor):  # type: ignore[override]
        group, n_local, world, rank, C, E, M = ctx.meta
        dst_rank, dst_row, flat, keep, w, saved = ctx.saved_tensors
        S = dst_rank.shape[0]
        dy = dy.contiguous()
        ws = symm.workspace_for(group) if (dy.is_cuda and comm.comm_mode() == "fused" and dy.dtype == torch.bfloat16) else None
        if ws is not None:
            # d(expert_out): gate-weighted rows of dy pushed into the owners' gradient buffers
            private = ctx.private
            gbuf = ctx.owner.bufs["grad"] if private else ws.scratch("moe_grad", (n_local * world * C, M), dy.dtype)
            if ctx.fill is None:
                gbuf.zero_()
            ws.moe_scatter_rows(gbuf, dy, dst_rank.view(-1), dst_row.view(-1), w.view(-1), 2, fill=ctx.fill)
            d_eo = gbuf.view(n_local, world * C, M)
            if not private:
                d_eo = d_eo.clone()
            # d(gate): <expert_out row, dy row>, read remotely
            if private:
                obuf = saved  # still in place since the forward
            else:
                obuf = ws.scratch("moe_out", (n_local * world * C, M), dy.dtype)
                obuf.copy_(saved.reshape(-1, M))
            dots = torch.zeros((S, 2), dtype=torch.float32, device=dy.device)
            ws.moe_gather_rows(obuf, None, dst_rank.view(-1), dst_row.view(-1), None, 2, grad=dy, dots=dots.view(-1))
            return d_eo, (dots * keep).to(w.dtype), None, None, None, None
        rows = saved  # [S, 2, M]
        d_gate = (rows.float() * dy.float().unsqueeze(1)).sum(-1) * keep
        contrib = dy.float().unsqueeze(1) * w.unsqueeze(-1)  # [S, 2, M]
        home = dy.new_zeros((E * C, M), dtype=torch.float32)
        for k in range(2):
            kept = keep[:, k]
            home.index_add_(0, flat[kept, k], contrib[kept, k])
        home = home.to(dy.dtype)
        back = torch.empty_like(home)
        comm.all_to_all_single(back, home, group)
        d_eo = back.view(world, n_local, C, M).transpose(0, 1).reshape(n_local, world * C, M)
        return d_eo, d_gate.to(w.dtype), None, None, None, None


class MOELayer(Base):
    """GShard mixture of experts: ``gate`` routes every token to two experts spread over ``group``.

    Args:
        gate: module returning ``(l_aux, combine_weights[S,E,C], dispatch_mask[S,E,C])``; gates that also have
            a ``route(x) -> Top2Route`` method take the index fast path.
        experts: one module or a ``ModuleList`` of this rank's local experts.
        group: expert-parallel process group (default WORLD).
    """

    def __init__(self, gate: Module, experts: Union[Module, ModuleList], group: Optional[Any] = None) -> None:
        super().__init__()
        self.gate = gate
        self._grouped = bool(getattr(experts, "grouped", False))  # stacked experts: one call for all of them
        self.experts = cast(ModuleList, experts) if type(experts) == ModuleList else ModuleList([experts])
        self.group = group if group is not None else dist.group.WORLD
        for expert in self.experts:
            for p in expert.parameters():
                p.expert = True  # type: ignore[attr-defined]  # data-parallel reducers must skip these
        self.world_size = dist.get_world_size(self.group)
        self.num_local_experts = len(experts) if self._grouped else len(self.experts)  # type: ignore[arg-type]
        self._heap_buffers = _LayerBuffers()

    def forward(self, *input: Tensor, **kwargs: Any) -> Tensor:
        assert len(input) == 1, "only single input Tensor supported"
        x = input[0]
        assert len(x.shape) == 3, "input Tensor must have dimensions: (s)equence, (t)oken, (m)odel"
        assert x.shape[0] % self.num_local_experts == 0, "num tokens must be order of number of local experts"
        d_model = x.shape[2]
        tokens = x.reshape(-1, d_model)

        if hasattr(self.gate, "route"):
            route: Top2Route = self.gate.route(tokens)
            self.l_aux = route.l_aux
            self._heap_buffers.expect_backward = torch.is_grad_enabled()
            expert_in = _Dispatch.apply(tokens, route, self.group, self.num_local_experts, self._heap_buffers)  # [n_local, world*C, M]
            if self._grouped:
                expert_out = self.experts[0](expert_in)  # every local expert in one grouped launch
            else:
                outs = []
                for e, expert in enumerate(self.experts):
                    chunk = expert_in[e].view(self.world_size, 1, route.capacity, d_model)
                    outs.append(expert(chunk).reshape(self.world_size * route.capacity, d_model))
                expert_out = torch.stack(outs, dim=0)
            combined = _Combine.apply(expert_out, route.gate, route, self.group, self.num_local_experts, self._heap_buffers)
            return combined.reshape(x.shape)

        self.l_aux, combine_weights, dispatch_mask = self.gate(tokens)
        dispatched = torch.einsum("sec,sm->ecm", dispatch_mask.to(tokens.dtype), tokens)
        dispatched = _AllToAll.apply(self.group, dispatched)
        dispatched = dispatched.reshape(self.world_size, self.num_local_experts, -1, d_model)
        if self._grouped:
            blk = dispatched.transpose(0, 1).reshape(self.num_local_experts, -1, d_model)
            expert_output = self.experts[0](blk).reshape(self.num_local_experts, self.world_size, -1, d_model).transpose(0, 1)
        else:
            chunks = dispatched.chunk(self.num_local_experts, dim=1)
            expert_outputs = [expert(chunk) for chunk, expert in zip(chunks, self.experts)]
            expert_output = torch.cat(expert_outputs, dim=1)
        expert_output = _AllToAll.apply(self.group, expert_output)
        expert_output = expert_output.reshape(self.world_size * self.num_local_experts, -1, d_model)
        combined = torch.einsum("sec,ecm->sm", combine_weights.to(tokens.dtype), expert_output)
        return combined.reshape(x.shape)
