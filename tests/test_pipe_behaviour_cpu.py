"""Pipe on CPU devices: it must be transparent (same outputs and gradients as the plain model for every chunking and
checkpoint mode), accept identity autograd functions and tuple inputs, cope with in-place ops and evaluation mode, and the
balance helpers must produce usable partitions."""
import copy

import pytest
import torch
from torch import nn

from fairscale_b200.nn.pipe import Pipe
from fairscale_b200.nn.pipe.balance import balance_by_size, balance_by_time


def _mlp():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(4, 8), nn.Tanh(), nn.Linear(8, 8), nn.Tanh(), nn.Linear(8, 2))


@pytest.mark.parametrize("chunks", [1, 2, 5])
@pytest.mark.parametrize("checkpoint", ["never", "except_last", "always"])
@pytest.mark.parametrize("balance", [[5], [2, 3], [1, 1, 1, 1, 1]])
def test_transparency(chunks, checkpoint, balance):
    plain = _mlp()
    piped = Pipe(copy.deepcopy(plain), balance, devices=["cpu"] * len(balance), chunks=chunks, checkpoint=checkpoint)
    x = torch.randn(5, 4)
    a, b = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, yb = plain(a), piped(b)
    torch.testing.assert_close(ya, yb)
    ya.pow(2).sum().backward()
    yb.pow(2).sum().backward()
    torch.testing.assert_close(a.grad, b.grad)
    for p, q in zip(plain.parameters(), piped.parameters()):
        torch.testing.assert_close(p.grad, q.grad)


def test_identity_autograd_function_and_tuple_flow():
    class Identity(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            return x

        @staticmethod
        def backward(ctx, g):
            return g

    class Id(nn.Module):
        def forward(self, x):
            return Identity.apply(x)

    pipe = Pipe(nn.Sequential(Id(), Id()), [1, 1], devices=["cpu", "cpu"], checkpoint="always")
    x = torch.rand(6, requires_grad=True)
    y = pipe(x)
    assert torch.allclose(x, y)
    y.sum().backward()
    assert torch.equal(x.grad, torch.ones(6))

    class Split(nn.Module):
        def forward(self, x):
            return x * 2, x + 1

    class Merge(nn.Module):
        def forward(self, ab):
            a, b = ab
            return a - b

    pipe = Pipe(nn.Sequential(Split(), Merge()), [1, 1], devices=["cpu", "cpu"], chunks=2)
    x = torch.arange(4.0).view(4, 1)
    torch.testing.assert_close(pipe(x), x - 1)


def test_inplace_relu_on_a_tensor_that_requires_grad_is_reported():
    pipe = Pipe(nn.Sequential(nn.Linear(1, 1), nn.ReLU(inplace=True)), [1, 1], devices=["cpu", "cpu"], checkpoint="always")
    y = pipe(torch.rand(1))
    with pytest.raises(RuntimeError, match="in-place"):
        y.backward()


def test_eval_mode_runs_without_checkpoints_or_graph():
    pipe = Pipe(_mlp(), [3, 2], devices=["cpu", "cpu"], chunks=2, checkpoint="always")
    pipe.eval()
    with torch.no_grad():
        y = pipe(torch.randn(4, 4))
    assert y.shape == (4, 2) and not y.requires_grad
    pipe.train()
    assert pipe(torch.randn(4, 4)).requires_grad


def test_exception_names_no_partial_results():
    class Boom(nn.Module):
        def forward(self, x):
            raise ValueError("bad layer")

    pipe = Pipe(nn.Sequential(nn.Identity(), Boom()), [1, 1], devices=["cpu", "cpu"], chunks=3)
    with pytest.raises(ValueError, match="bad layer"):
        pipe(torch.randn(3, 2))
    # the pipe is usable again afterwards
    ok = Pipe(nn.Sequential(nn.Identity(), nn.Identity()), [1, 1], devices=["cpu", "cpu"], chunks=3)
    assert ok(torch.ones(3, 2)).sum() == 6


def test_balance_helpers_give_valid_partitions():
    model = _mlp()
    sample = torch.randn(8, 4)
    by_time = balance_by_time(2, model, sample, timeout=0.2, device=torch.device("cpu"))
    assert sum(by_time) == len(model) and len(by_time) == 2 and all(b > 0 for b in by_time)
    Pipe(model, by_time, devices=["cpu"] * 2)(sample)
    with pytest.raises(ValueError, match="CUDA"):  # the size profiler reads the CUDA allocator, as in the reference
        balance_by_size(3, model, sample, chunks=2, param_scale=2.0, device=torch.device("cpu"))
