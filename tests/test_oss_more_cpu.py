"""More OSS behaviours on gloo CPU ranks (cases of the reference's tests/optim/test_oss.py): optimizers that add keys to their
parameter groups or take no closure, asking for the state dict before it was consolidated, more ranks than parameters,
balanced partitions, ``state_dict(all_ranks=True)`` on every rank, reproducibility after reloading a checkpoint (also with fp16
broadcasts), a changing training graph against DistributedDataParallel, and ``zero_grad``."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.optim import OSS


def _net(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(5, 8), nn.Tanh(), nn.Linear(8, 8), nn.Tanh(), nn.Linear(8, 3))


def _batch(rank, step):
    g = torch.Generator().manual_seed(13 * step + rank)
    return torch.randn(6, 5, generator=g), torch.randn(6, 3, generator=g)


def _all_reduce_grads(model, world):
    for p in model.parameters():
        if p.grad is not None:
            dist.all_reduce(p.grad)
            p.grad /= world


def _inner_optimizer_quirks(rank, world):
    class AddsAKey(torch.optim.SGD):
        def step(self, closure=None):
            super().step()
            self.param_groups[0]["new_key"] = 0.1  # must show up in the outer groups after the step

    class NoClosure(torch.optim.SGD):
        def step(self):  # type: ignore[override]
            return super().step()

    for cls in (AddsAKey, NoClosure):
        x = torch.tensor([1.0], requires_grad=True)
        o = OSS([x], cls, lr=0.1)
        x.backward()
        o.step()
        assert torch.allclose(x.detach(), torch.tensor([0.9]))
        if cls is AddsAKey:
            assert o.param_groups[0]["new_key"] == 0.1

    # the state of the other ranks is not here until consolidate_state_dict() has run
    x = torch.tensor([1.0], requires_grad=True)
    o = OSS([x], lr=0.1)
    with pytest.raises(RuntimeError):
        o.state_dict()
    # zero_grad: to zero, or to None
    x.backward()
    o.zero_grad(set_to_none=False)
    assert x.grad is not None and float(x.grad) == 0.0
    o.zero_grad(set_to_none=True)
    assert x.grad is None


def test_oss_inner_optimizer_quirks_and_unconsolidated_state_dict():
    spawn_ranks(_inner_optimizer_quirks, 1, (), backend="gloo")


def _more_ranks_than_parameters(rank, world):
    """Two parameters over four ranks: two ranks own nothing, step / state-dict / clipping still work everywhere."""
    torch.manual_seed(0)
    m = nn.Linear(1, 1)
    o = OSS(m.parameters(), lr=0.1, momentum=0.5)
    owned = sum(len(g["params"]) for g in o.optim.param_groups)
    counts = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(counts, torch.tensor([float(owned)]))
    assert sorted(int(c) for c in counts) == [0, 0, 1, 1]
    for step in range(2):
        m.zero_grad()
        m(torch.full((1,), float(rank + 1))).backward()
        _all_reduce_grads(m, world)
        o.clip_grad_norm(1.0)
        o.step()
    o.consolidate_state_dict(recipient_rank=0)
    if rank == 0:
        assert len(o.state_dict()["state"]) == 2
    weights = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(weights, m.weight.detach().reshape(1))
    assert all(torch.equal(weights[0], w) for w in weights)


def test_oss_with_more_ranks_than_parameters():
    spawn_ranks(_more_ranks_than_parameters, 4, (), backend="gloo")


def _balanced_partitions(rank, world):
    """Sizes 9, 7, 5, 3 repeated per rank: the greedy size-balanced partition gives every rank the same number of elements."""
    sizes = [9, 7, 5, 3] * world
    params = [torch.rand(s, 1, requires_grad=True) for s in sizes]
    o = OSS(params, lr=0.1)
    mine = sum(p.numel() for g in o.optim.param_groups for p in g["params"])
    assert mine == sum(sizes) // world, (mine, sum(sizes) // world)
    # every parameter has exactly one owner
    ranks = sorted(o._param_to_rank[p] for p in params)
    assert ranks == sorted(list(range(world)) * 4)


def test_oss_partitions_are_balanced_by_size():
    spawn_ranks(_balanced_partitions, 4, (), backend="gloo")


def _reload(rank, world, broadcast_fp16):
    """Train, checkpoint (consolidated on rank 0, shipped to everybody), train on; restore and train again: the same loss."""
    model = _net()
    o = OSS(model.parameters(), optim=torch.optim.RMSprop, lr=0.01, broadcast_fp16=broadcast_fp16)

    def one_step(step):
        x, y = _batch(0, step)  # the same data on every rank: local gradients are the global ones
        o.zero_grad()
        loss = nn.functional.mse_loss(model(x), y)
        loss.backward()
        o.step()
        return float(loss)

    one_step(0)
    o.consolidate_state_dict(recipient_rank=0)
    box = [copy.deepcopy(o.state_dict()) if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    weights = copy.deepcopy(model.state_dict())
    first = [one_step(1), one_step(2)]

    model.load_state_dict(weights)
    o.load_state_dict(box[0])
    again = [one_step(1), one_step(2)]
    tol = 5e-3 if broadcast_fp16 else 1e-6  # fp16 broadcasts round the weights every rank receives
    assert all(abs(a - b) <= tol * max(1.0, abs(a)) for a, b in zip(first, again)), (first, again)

    # the global state materialised on every rank at once (no recipient), and loaded back
    everywhere = o.state_dict(all_ranks=True)
    assert len(everywhere["state"]) == len(list(model.parameters()))
    o.load_state_dict(everywhere)
    one_step(3)


@pytest.mark.parametrize("broadcast_fp16", [False, True])
def test_oss_training_is_reproducible_after_reloading_a_checkpoint(broadcast_fp16):
    spawn_ranks(_reload, 2, (broadcast_fp16,), backend="gloo")


def _changing_graph(rank, world, broadcast_fp16):
    """Against DistributedDataParallel + the plain optimizer while layers are frozen and thawed between steps (OSS has to
    re-partition what it updates and what it broadcasts)."""
    ref_model, model = _net(), _net()
    ref = nn.parallel.DistributedDataParallel(ref_model, find_unused_parameters=True)
    ref_opt = torch.optim.SGD(ref_model.parameters(), lr=0.05, momentum=0.9)
    o = OSS(model.parameters(), optim=torch.optim.SGD, lr=0.05, momentum=0.9, broadcast_fp16=broadcast_fp16)
    for step in range(6):
        if step in (2, 4):
            freeze = step == 2
            for net in (ref_model, model):
                for p in net[2].parameters():
                    p.requires_grad = not freeze
                    if freeze:
                        p.grad = None
            o.refresh_trainable()
        x, y = _batch(rank, step)
        ref_opt.zero_grad()
        nn.functional.mse_loss(ref(x), y).backward()
        ref_opt.step()
        o.zero_grad(set_to_none=True)
        nn.functional.mse_loss(model(x), y).backward()
        _all_reduce_grads(model, world)
        o.step()
    tol = dict(atol=2e-3, rtol=2e-2) if broadcast_fp16 else dict(atol=1e-6, rtol=1e-5)
    for a, b in zip(ref_model.parameters(), model.parameters()):
        torch.testing.assert_close(b, a, **tol)


@pytest.mark.parametrize("broadcast_fp16", [False, True])
def test_oss_matches_ddp_while_the_training_graph_changes(broadcast_fp16):
    spawn_ranks(_changing_graph, 2, (broadcast_fp16,), backend="gloo")
