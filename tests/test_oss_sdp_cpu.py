"""OSS and ShardedDataParallel behaviours on gloo CPU ranks: state-dict consolidation and cross-loading with a plain
optimizer, gradient clipping, added parameter groups, gradient accumulation under ``no_sync``, frozen parameters and an
uneven world (3 ranks, fewer large parameters than ranks)."""
import copy

import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.data_parallel import ShardedDataParallel
from fairscale_b200.optim import OSS


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(6, 11), nn.Tanh(), nn.Linear(11, 5), nn.Tanh(), nn.Linear(5, 3))


def _batch(rank, step, n=4):
    g = torch.Generator().manual_seed(1000 * step + rank)
    return torch.randn(n, 6, generator=g), torch.randn(n, 3, generator=g)


def _step(model, opt, rank, step, clip=None, oss=None):
    x, y = _batch(rank, step)
    # gradients of a ShardedDataParallel module are views of its reduce buckets: they are cleared through the module
    model.zero_grad() if isinstance(model, ShardedDataParallel) else opt.zero_grad()
    loss = nn.functional.mse_loss(model(x), y)
    loss.backward()
    norm = None
    if clip is not None:
        norm = oss.clip_grad_norm(clip) if oss is not None else torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
    opt.step()
    return loss.item(), norm


def _state_and_clip(rank, world):
    ref = nn.parallel.DistributedDataParallel(_model())
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    base = _model()
    oss = OSS(base.parameters(), optim=torch.optim.SGD, lr=0.1, momentum=0.9)
    sdp = ShardedDataParallel(base, oss)

    # every parameter is owned by exactly one rank
    owned = [sum(len(g["params"]) for g in part) for part in oss.partition_parameters()]
    assert sum(owned) == len(list(base.parameters())) and len(owned) == world

    for s in range(3):
        l_ref, n_ref = _step(ref, ref_opt, rank, s, clip=0.5)
        l_new, n_new = _step(sdp, oss, rank, s, clip=0.5, oss=oss)
        assert abs(l_ref - l_new) < 1e-6
        torch.testing.assert_close(torch.as_tensor(n_new).float(), torch.as_tensor(n_ref).float(), atol=1e-5, rtol=1e-5)
    for a, b in zip(ref.module.parameters(), base.parameters()):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)

    # consolidated state on rank 0 has the layout of the plain optimizer's state dict and loads into one
    oss.consolidate_state_dict(recipient_rank=0)
    if rank == 0:
        full = oss.state_dict()
        ref_sd = ref_opt.state_dict()
        assert len(full["state"]) == len(ref_sd["state"])
        for pid, st in ref_sd["state"].items():
            torch.testing.assert_close(full["state"][pid]["momentum_buffer"], st["momentum_buffer"], atol=1e-6, rtol=1e-5)
        plain = torch.optim.SGD(_model().parameters(), lr=0.1, momentum=0.9)
        plain.load_state_dict(full)
        box = [full]
    else:
        box = [None]
    dist.broadcast_object_list(box, src=0)

    # a plain optimizer's state dict loads into a fresh OSS: each rank keeps its shard and training continues in step
    base2 = copy.deepcopy(base)
    oss2 = OSS(base2.parameters(), optim=torch.optim.SGD, lr=0.1, momentum=0.9)
    oss2.load_state_dict(box[0])
    sdp2 = ShardedDataParallel(base2, oss2)
    l_ref, _ = _step(ref, ref_opt, rank, 7)
    l_new, _ = _step(sdp2, oss2, rank, 7)
    assert abs(l_ref - l_new) < 1e-6
    for a, b in zip(ref.module.parameters(), base2.parameters()):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)

    # local (non-consolidated) state dict exists on every rank without communication
    local = oss.optim.state_dict()
    assert len(local["state"]) == owned[rank]


def test_oss_state_dict_clip_and_cross_loading():
    spawn_ranks(_state_and_clip, 2, (), backend="gloo")


def _accumulate_freeze_add_group(rank, world):
    ref = nn.parallel.DistributedDataParallel(_model())
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    base = _model()
    oss = OSS(base.parameters(), optim=torch.optim.SGD, lr=0.05)
    sdp = ShardedDataParallel(base, oss, reduce_buffer_size=0)

    # two micro-batches without reduction, one with: same update as DDP's no_sync accumulation
    ref_opt.zero_grad()
    sdp.zero_grad()
    for s in range(3):
        x, y = _batch(rank, s)
        if s < 2:
            with ref.no_sync():
                nn.functional.mse_loss(ref(x), y).backward()
            with sdp.no_sync():
                nn.functional.mse_loss(sdp(x), y).backward()
        else:
            nn.functional.mse_loss(ref(x), y).backward()
            nn.functional.mse_loss(sdp(x), y).backward()
    ref_opt.step()
    oss.step()
    for a, b in zip(ref.module.parameters(), base.parameters()):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)

    # freeze the first layer: refresh_trainable() rebuilds the hooks and the frozen weights stay put
    for p in base[0].parameters():
        p.requires_grad = False
        p.grad = None  # the module's zero_grad only visits trainable parameters, as in the reference
    sdp.refresh_trainable()
    frozen = [p.detach().clone() for p in base[0].parameters()]
    before = base[4].weight.detach().clone()
    _step(sdp, oss, rank, 5)
    assert all(torch.equal(a, b) for a, b in zip(frozen, base[0].parameters()))
    assert not torch.equal(before, base[4].weight)
    ranks_agree = [torch.zeros_like(base[4].weight) for _ in range(world)]
    dist.all_gather(ranks_agree, base[4].weight.detach())
    assert all(torch.equal(ranks_agree[0], t) for t in ranks_agree)  # owners broadcast the update to everyone

    # a parameter group added later is partitioned too
    extra = nn.Linear(3, 3)
    oss.add_param_group({"params": list(extra.parameters()), "lr": 0.01})
    assert len(oss.param_groups) == 2
    assert sum(len(g["params"]) for part in oss.partition_parameters() for g in part) == len(list(base.parameters())) + 2


def test_sdp_accumulation_freezing_and_new_groups():
    spawn_ranks(_accumulate_freeze_add_group, 2, (), backend="gloo")


def _uneven(rank, world):
    # three ranks, a model with two big tensors and a few tiny ones: some rank owns only small parameters
    ref = nn.parallel.DistributedDataParallel(_model())
    ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-2)
    base = _model()
    oss = OSS(base.parameters(), optim=torch.optim.Adam, lr=1e-2)
    sdp = ShardedDataParallel(base, oss)
    for s in range(3):
        l_ref, _ = _step(ref, ref_opt, rank, s)
        l_new, _ = _step(sdp, oss, rank, s)
        assert abs(l_ref - l_new) < 1e-6
    for a, b in zip(ref.module.parameters(), base.parameters()):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)


def test_oss_sdp_three_ranks():
    spawn_ranks(_uneven, 3, (), backend="gloo")


def _two_optimizers_manual_reduce_buffers(rank, world):
    # two sharded optimizers over disjoint halves of one module, as one ShardedDataParallel
    torch.manual_seed(0)
    base = nn.Sequential(nn.Linear(6, 8), nn.BatchNorm1d(8), nn.Tanh(), nn.Linear(8, 3))
    ref = nn.parallel.DistributedDataParallel(copy.deepcopy(base), broadcast_buffers=True)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    first = OSS(list(base[0].parameters()) + list(base[1].parameters()), optim=torch.optim.SGD, lr=0.05)
    second = OSS(base[3].parameters(), optim=torch.optim.SGD, lr=0.05)
    sdp = ShardedDataParallel(base, [first, second])
    for s in range(3):
        x, y = _batch(rank, s)
        ref_opt.zero_grad()
        nn.functional.mse_loss(ref(x), y).backward()
        ref_opt.step()
        sdp.zero_grad()
        nn.functional.mse_loss(sdp(x), y).backward()
        first.step()
        second.step()
    for a, b in zip(ref.module.parameters(), base.parameters()):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)

    # manual reduction after no_sync accumulation
    sdp.zero_grad()
    x, y = _batch(rank, 9)
    with sdp.no_sync():
        nn.functional.mse_loss(sdp(x), y).backward()
    local = base[3].weight.grad.clone() if base[3].weight.grad is not None else None
    sdp.reduce()
    owner = second._param_to_rank[base[3].weight]
    # every rank contributes its local gradient; the owner ends up with the mean
    contrib = local if local is not None else torch.zeros_like(base[3].weight)
    allg = [torch.zeros_like(contrib) for _ in range(world)]
    dist.all_gather(allg, contrib)
    if rank == owner:
        torch.testing.assert_close(base[3].weight.grad, sum(allg) / world, atol=1e-6, rtol=1e-5)

    # buffers: diverge on one rank, sync_buffers brings rank 0's statistics back everywhere
    if rank == 1:
        base[1].running_mean.add_(5.0)
    sdp.sync_buffers(blocking=True)
    means = [torch.zeros_like(base[1].running_mean) for _ in range(world)]
    dist.all_gather(means, base[1].running_mean)
    assert all(torch.equal(means[0], m) for m in means)

    # evaluation forward does not touch the gradient machinery
    sdp.eval()
    with torch.no_grad():
        out = sdp(x)
    assert not out.requires_grad
    sdp.train()


def test_sdp_two_optimizers_manual_reduce_and_buffers():
    spawn_ranks(_two_optimizers_manual_reduce_buffers, 2, (), backend="gloo")


class _SGDWithKwarg(torch.optim.SGD):
    def step(self, closure=None, kwarg=None):
        super().step()
        kwarg.append(5)


def _oss_optimizer_protocol(rank, world):
    # closure, extra step kwargs, lr schedulers and param-group edits pass through the sharded wrapper
    x = torch.tensor([float(rank + 1)])
    m = nn.Linear(1, 1)
    with torch.no_grad():
        m.weight.fill_(1.0)
        m.bias.fill_(2.0)
    o = OSS(m.parameters(), optim=torch.optim.SGD, lr=0.1)

    def closure():
        o.zero_grad()
        loss = (m(x) - 0.0).pow(2).sum()
        loss.backward()
        return loss

    loss = o.step(closure=closure)
    assert loss is not None and float(loss) == (rank + 1 + 2) ** 2
    # every rank ends with the owners' values (here every rank fed a different input: the owner's update wins)
    w = [torch.zeros_like(m.weight) for _ in range(world)]
    dist.all_gather(w, m.weight.detach())
    assert all(torch.equal(w[0], t) for t in w)

    seen = []
    o2 = OSS(nn.Linear(1, 1).parameters(), optim=_SGDWithKwarg, lr=0.1)
    o2.step(kwarg=seen)  # forwarded to the wrapped optimizer
    assert seen == [5]

    sched = torch.optim.lr_scheduler.StepLR(o, step_size=1, gamma=0.5)
    o.step()
    sched.step()
    assert abs(o.param_groups[0]["lr"] - 0.05) < 1e-12
    o.step()  # the local optimizer sees the new learning rate
    assert abs(o.optim.param_groups[0]["lr"] - 0.05) < 1e-12

    # a process group that is not the world: ranks {0, 1} of three shard among themselves
    sub = dist.new_group(ranks=[0, 1])
    if rank < 2:
        m3 = nn.Sequential(nn.Linear(2, 2), nn.Linear(2, 2))
        o3 = OSS(m3.parameters(), optim=torch.optim.SGD, group=sub, lr=0.1)
        assert len(o3.partition_parameters()) == 2
        m3(torch.ones(1, 2)).sum().backward()
        o3.step()
        vals = [torch.zeros_like(m3[1].bias) for _ in range(2)]
        dist.all_gather(vals, m3[1].bias.detach(), group=sub)
        assert torch.equal(vals[0], vals[1])
    dist.barrier()


def test_oss_closure_kwargs_scheduler_and_subgroup():
    spawn_ranks(_oss_optimizer_protocol, 3, (), backend="gloo")


def _bucketed_with_optimizer_zero_grad(rank, world):
    # the optimizer's zero_grad drops the gradients (set_to_none): autograd then produces private tensors, which the
    # wrapper moves back into the reduce bucket before the bucket is sent
    from torch.nn.parallel import DistributedDataParallel as DDP

    ref = DDP(_model())
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    base = _model()
    oss = OSS(base.parameters(), optim=torch.optim.SGD, lr=0.1, momentum=0.9)
    sdp = ShardedDataParallel(base, oss, reduce_buffer_size=2**20)
    for step in range(4):
        x, y = _batch(rank, step)
        ref_opt.zero_grad()
        nn.functional.mse_loss(ref(x), y).backward()
        ref_opt.step()
        oss.zero_grad()
        nn.functional.mse_loss(sdp(x), y).backward()
        oss.step()
    assert any(sdp._should_bucket_grad)
    for a, b in zip(ref.module.parameters(), base.parameters()):
        torch.testing.assert_close(b, a, atol=1e-6, rtol=1e-5)


def test_sdp_buckets_survive_optimizer_zero_grad():
    spawn_ranks(_bucketed_with_optimizer_zero_grad, 2, (), backend="gloo")
