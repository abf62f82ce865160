"""Sequence-parallel linears on gloo ranks (unfused path): forward and gradients equal the dense computation."""
import torch
import torch.distributed as dist

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.parallel.fused_tp import all_gather_linear, linear_reduce_scatter


def _worker(rank, world):
    torch.manual_seed(0)
    T, K, H, N = 8, 6, 10, 4
    x_full = torch.randn(T, K)
    w1 = torch.randn(H, K)          # column-parallel: split H
    b1 = torch.randn(H)
    w2 = torch.randn(N, H)          # row-parallel: split H
    b2 = torch.randn(N)
    xr = x_full.clone().requires_grad_()
    ref = torch.relu(xr @ w1.t() + b1) @ w2.t() + b2
    ref.pow(2).sum().backward()

    hs = H // world
    w1l = w1[rank * hs : (rank + 1) * hs].clone().requires_grad_()
    b1l = b1[rank * hs : (rank + 1) * hs].clone().requires_grad_()
    w2l = w2[:, rank * hs : (rank + 1) * hs].clone().requires_grad_()
    b2l = b2.clone().requires_grad_()
    ts = T // world
    xs = x_full[rank * ts : (rank + 1) * ts].clone().requires_grad_()
    h = torch.relu(all_gather_linear(xs, w1l, b1l))
    out = linear_reduce_scatter(h, w2l, b2l)
    torch.testing.assert_close(out, ref[rank * ts : (rank + 1) * ts].detach(), rtol=1e-4, atol=1e-4)
    out.pow(2).sum().backward()
    torch.testing.assert_close(xs.grad, xr.grad[rank * ts : (rank + 1) * ts], rtol=1e-4, atol=1e-4)
    w1f = w1.clone().requires_grad_(); b1f = b1.clone().requires_grad_(); w2f = w2.clone().requires_grad_(); b2f = b2.clone().requires_grad_()
    (torch.relu(x_full @ w1f.t() + b1f) @ w2f.t() + b2f).pow(2).sum().backward()
    torch.testing.assert_close(w1l.grad, w1f.grad[rank * hs : (rank + 1) * hs], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(b1l.grad, b1f.grad[rank * hs : (rank + 1) * hs], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(w2l.grad, w2f.grad[:, rank * hs : (rank + 1) * hs], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(b2l.grad, b2f.grad, rtol=1e-4, atol=1e-4)


def test_sequence_parallel_linears_match_dense():
    spawn_ranks(_worker, 2, (), backend="gloo")


def _all_reduce_worker(rank, world):
    from fairscale_b200.parallel.fused_tp import linear_all_reduce

    torch.manual_seed(0)
    T, H, N = 8, 10, 4
    h_full = torch.randn(T, H)
    w = torch.randn(N, H)
    b = torch.randn(N)
    hs = H // world
    hl = h_full[:, rank * hs : (rank + 1) * hs].clone().requires_grad_()
    wl = w[:, rank * hs : (rank + 1) * hs].clone().requires_grad_()
    bl = b.clone().requires_grad_()
    out = linear_all_reduce(hl, wl, bl)
    hr, wr, br = h_full.clone().requires_grad_(), w.clone().requires_grad_(), b.clone().requires_grad_()
    ref = hr @ wr.t() + br
    torch.testing.assert_close(out, ref.detach(), rtol=1e-4, atol=1e-4)
    g = torch.randn(T, N)  # the same upstream gradient on every rank (seeded above)
    out.backward(g)
    ref.backward(g)
    torch.testing.assert_close(hl.grad, hr.grad[:, rank * hs : (rank + 1) * hs], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(wl.grad, wr.grad[:, rank * hs : (rank + 1) * hs], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(bl.grad, br.grad, rtol=1e-4, atol=1e-4)


def test_row_parallel_product_with_fully_reduced_output():
    spawn_ranks(_all_reduce_worker, 2, (), backend="gloo")
