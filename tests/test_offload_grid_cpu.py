"""OffloadModel over the grid of the reference's tests/experimental/nn/test_offload.py::test_correctness (which the reference
keeps skipped): activation checkpointing on or off, one or five micro-batches, slices cut from a sequential model or produced
by ``shard_model`` from a model with a residual connection, under CPU autocast or not - against the same model trained
without offloading.  Also: slice counts that do not divide the layers, eval mode, and the state dict keys of the wrapper."""
import contextlib
import copy

import pytest
import torch
from torch import nn

from fairscale_b200.experimental.nn import OffloadModel
from fairscale_b200.experimental.nn.auto_shard import shard_model

CPU = torch.device("cpu")


def _sequential(layers=10, hidden=20):
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(2, hidden), *[nn.Linear(hidden, hidden) for _ in range(layers)], nn.Linear(hidden, 2))


class _Residual(nn.Module):
    def __init__(self, hidden=12):
        super().__init__()
        torch.manual_seed(0)
        self.inp = nn.Linear(2, hidden)
        self.a, self.b, self.c = nn.Linear(hidden, hidden), nn.Linear(hidden, hidden), nn.Linear(hidden, hidden)
        self.out = nn.Linear(hidden, 2)

    def forward(self, x):
        h = torch.tanh(self.inp(x))
        h = h + self.b(torch.tanh(self.a(h)))
        return self.out(torch.tanh(self.c(h)))


def _train(model, optimizer, autocast, steps=3):
    x, y = torch.ones(30, 2), torch.ones(30, 2)
    losses = []
    model.train()
    for _ in range(steps):
        ctx = torch.autocast("cpu", dtype=torch.bfloat16) if autocast else contextlib.nullcontext()
        with ctx:
            loss = nn.functional.mse_loss(model(x).float(), y, reduction="sum")
        loss.backward()
        optimizer.step()
        optimizer.zero_grad()
        losses.append(float(loss))
    return losses


@pytest.mark.parametrize("autocast", [False, True])
@pytest.mark.parametrize("checkpoint,microbatches", [(False, 1), (True, 1), (True, 5)])
@pytest.mark.parametrize("auto_shard", [False, True])
def test_training_matches_the_model_without_offloading(autocast, checkpoint, microbatches, auto_shard):
    plain = _Residual() if auto_shard else _sequential()
    twin = copy.deepcopy(plain)
    slices = shard_model(twin, 3) if auto_shard else twin
    offloaded = OffloadModel(model=slices, device=CPU, offload_device=CPU, num_slices=2 if not auto_shard else len(slices),
                             checkpoint_activation=checkpoint, num_microbatches=microbatches)
    want = _train(plain, torch.optim.SGD(plain.parameters(), lr=0.001), autocast)
    got = _train(offloaded, torch.optim.SGD(offloaded.parameters(), lr=0.001), autocast)
    tol = 2e-2 if autocast else 1e-5
    assert all(abs(a - b) <= tol * max(1.0, abs(b)) for a, b in zip(got, want)), (got, want)
    assert got[-1] < got[0]
    for a, b in zip(offloaded.parameters(), plain.parameters()):
        torch.testing.assert_close(a, b, atol=1e-2 if autocast else 1e-6, rtol=1e-2 if autocast else 1e-5)


@pytest.mark.parametrize("slices", [1, 3, 5, 12])
def test_slice_counts_that_do_not_divide_the_layers(slices):
    model = _sequential()
    offloaded = OffloadModel(copy.deepcopy(model), CPU, CPU, num_slices=slices)
    assert 1 <= len(offloaded.model_slices) <= slices
    assert sum(len(list(s.parameters())) for s in offloaded.model_slices) == len(list(model.parameters()))
    x = torch.randn(4, 2)
    torch.testing.assert_close(offloaded(x), model(x))
    offloaded.eval()
    with torch.no_grad():
        torch.testing.assert_close(offloaded(x), model(x))


def test_more_micro_batches_need_checkpointing_and_lists_are_taken_as_slices():
    with pytest.raises(RuntimeError):
        OffloadModel(_sequential(), CPU, CPU, num_slices=2, checkpoint_activation=False, num_microbatches=5)
    with pytest.raises(TypeError):
        OffloadModel(_Residual(), CPU, CPU)  # neither sequential nor a list of slices
    pieces = shard_model(_Residual(), 2)
    offloaded = OffloadModel(pieces, CPU, CPU)
    assert len(offloaded.model_slices) == len(pieces)
    assert offloaded(torch.randn(3, 2)).shape == (3, 2)
