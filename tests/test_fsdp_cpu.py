"""FSDP on gloo CPU ranks: parity with DDP, state-dict formats, optimizer-state consolidation, no_sync, clipping."""
import copy
import functools
import itertools
import pickle

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import DummyProcessGroup, spawn_ranks
from fairscale_b200.nn import FullyShardedDataParallel as FSDP
from fairscale_b200.nn import auto_wrap, default_auto_wrap_policy, enable_wrap, wrap
from fairscale_b200.nn.data_parallel import TrainingState, get_fsdp_instances
from fairscale_b200.parallel import comm


class Net(nn.Module):
    """Nested model with an odd-sized layer so shards need padding and a shared (tied) weight inside one unit."""

    def __init__(self, wrap_inner=None, d=16):
        super().__init__()
        torch.manual_seed(0)
        w = wrap_inner or (lambda m: m)
        self.embed = nn.Embedding(23, d)
        self.block1 = w(nn.Sequential(nn.Linear(d, 3 * d + 1), nn.GELU(), nn.Linear(3 * d + 1, d)))
        self.block2 = w(nn.Sequential(nn.LayerNorm(d), nn.Linear(d, d)))
        self.head = nn.Linear(d, 23, bias=False)
        self.head.weight = self.embed.weight  # tied

    def forward(self, tokens):
        h = self.embed(tokens)
        h = h + self.block1(h)
        h = h + self.block2(h)
        return self.head(h)


def _loss(model, tokens):
    out = model(tokens)
    return nn.functional.cross_entropy(out.float().view(-1, out.size(-1)), tokens.view(-1))


def _data(rank, step):
    g = torch.Generator().manual_seed(100 * step + rank)
    return torch.randint(0, 23, (4, 7), generator=g)


def _train(model, opt, rank, steps=3, clip=None):
    losses = []
    for s in range(steps):
        opt.zero_grad()
        loss = _loss(model, _data(rank, s))
        loss.backward()
        if clip is not None:
            if isinstance(model, FSDP):
                model.clip_grad_norm_(clip)
            else:
                torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
        opt.step()
        losses.append(loss.item())
    return losses


def _parity(rank, world, reshard, flatten, nested, mixed, clip):
    ref = nn.parallel.DistributedDataParallel(Net())
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    ref_losses = _train(ref, ref_opt, rank, clip=clip)

    kw = dict(reshard_after_forward=reshard, flatten_parameters=flatten, mixed_precision=mixed,
              compute_device=torch.device("cpu"), compute_dtype=torch.bfloat16 if mixed else None)
    inner = (lambda m: FSDP(m, **kw)) if nested else None
    model = FSDP(Net(inner), **kw)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    losses = _train(model, opt, rank, clip=clip)
    tol = dict(atol=5e-2, rtol=5e-2) if mixed else dict(atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(torch.tensor(losses), torch.tensor(ref_losses), **tol)
    full = model.state_dict()
    ref_sd = ref.module.state_dict()
    assert set(full.keys()) == set(ref_sd.keys()), (sorted(full.keys()), sorted(ref_sd.keys()))
    for k in ref_sd:
        torch.testing.assert_close(full[k], ref_sd[k], **tol)
    for m in get_fsdp_instances(model):
        assert m.training_state == TrainingState.IDLE


@pytest.mark.parametrize("reshard,flatten,nested", list(itertools.product([True, False], [True, False], [True, False])))
def test_fsdp_matches_ddp(reshard, flatten, nested):
    if not flatten and True:
        # tied weights need one flat parameter (or append_shared_param); covered by the flatten cases
        pytest.skip("tied weight requires flatten_parameters")
    spawn_ranks(_parity, 2, (reshard, flatten, nested, False, None), backend="gloo")


def test_fsdp_mixed_precision_and_clip():
    spawn_ranks(_parity, 2, (True, True, True, True, None), backend="gloo")
    spawn_ranks(_parity, 2, (True, True, True, False, 0.05), backend="gloo")


class Plain(nn.Module):
    def __init__(self, wrap_inner=None, d=12):
        super().__init__()
        torch.manual_seed(1)
        w = wrap_inner or (lambda m: m)
        self.a = w(nn.Linear(d, 2 * d + 1))
        self.b = w(nn.Linear(2 * d + 1, d))
        self.register_buffer("scale", torch.ones(1))

    def forward(self, x):
        return self.b(torch.relu(self.a(x))) * self.scale


def _unflat_parity(rank, world):
    ref = nn.parallel.DistributedDataParallel(Plain())
    ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-2)
    kw = dict(flatten_parameters=False, compute_device=torch.device("cpu"))
    model = FSDP(Plain(lambda m: FSDP(m, **kw)), **kw)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    for s in range(3):
        x = torch.randn(5, 12, generator=torch.Generator().manual_seed(10 * s + rank))
        for mdl, o in ((ref, ref_opt), (model, opt)):
            o.zero_grad()
            mdl(x).pow(2).mean().backward()
            o.step()
    sd, ref_sd = model.state_dict(), ref.module.state_dict()
    assert set(sd) == set(ref_sd)
    for k in sd:
        torch.testing.assert_close(sd[k], ref_sd[k], atol=1e-5, rtol=1e-5)


def test_fsdp_unflattened_matches_ddp():
    spawn_ranks(_unflat_parity, 2, (), backend="gloo")


def _state_roundtrip(rank, world, tmpdir):
    kw = dict(compute_device=torch.device("cpu"))
    model = FSDP(Net(lambda m: FSDP(m, **kw)), **kw)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    _train(model, opt, rank, steps=2)
    full = model.state_dict()

    # local shards + metadata -> consolidated full weights, offline
    torch.save(model.local_state_dict(), f"{tmpdir}/w{rank}.pt")
    torch.save(model.local_metadata_dict(), f"{tmpdir}/m{rank}.pt")
    dist.barrier()
    if rank == 0:
        ws = [torch.load(f"{tmpdir}/w{r}.pt", weights_only=False) for r in range(world)]
        ms = [torch.load(f"{tmpdir}/m{r}.pt", weights_only=False) for r in range(world)]
        merged = FSDP.consolidate_shard_weights(ws, ms)
        assert set(merged) == set(full), (sorted(merged), sorted(full))
        for k in full:
            torch.testing.assert_close(merged[k], full[k])
        bare = Net()
        bare.load_state_dict(merged)

    # local state dict round trip
    local = copy.deepcopy(model.local_state_dict())
    assert any(k.endswith("flat_param_0") for k in local), list(local)
    with torch.no_grad():
        for p in model.parameters():
            p.add_(1.0)
    model.load_local_state_dict(local)
    after = model.state_dict()
    for k in full:
        torch.testing.assert_close(after[k], full[k])

    # full state dict round trip into a fresh wrapper
    fresh = FSDP(Net(lambda m: FSDP(m, **kw)), **kw)
    with torch.no_grad():
        for p in fresh.parameters():
            p.zero_()
    fresh.load_state_dict(full)
    again = fresh.state_dict()
    for k in full:
        torch.testing.assert_close(again[k], full[k])

    # optimizer state: gather on rank 0, compare with the unwrapped run, re-shard and resume
    osd = model.gather_full_optim_state_dict(opt)
    ref = nn.parallel.DistributedDataParallel(Net())
    ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-2)
    _train(ref, ref_opt, rank, steps=2)
    box = [osd]
    dist.broadcast_object_list(box, src=0)
    osd = box[0]
    ref_osd = ref_opt.state_dict()
    assert len(osd["state"]) == len(ref_osd["state"])
    for pid, st in ref_osd["state"].items():
        torch.testing.assert_close(osd["state"][pid]["exp_avg"], st["exp_avg"], atol=1e-6, rtol=1e-5)
        assert osd["state"][pid]["exp_avg"].shape == st["exp_avg"].shape
    shard = model.get_shard_from_optim_state_dict(copy.deepcopy(osd))
    opt2 = torch.optim.Adam(model.parameters(), lr=1e-2)
    opt2.load_state_dict(shard)
    for pid, st in opt.state_dict()["state"].items():
        torch.testing.assert_close(opt2.state_dict()["state"][pid]["exp_avg"], st["exp_avg"])


def test_fsdp_state_dict_formats(tmp_path):
    spawn_ranks(_state_roundtrip, 2, (str(tmp_path),), backend="gloo")


def _no_sync_and_summon(rank, world):
    kw = dict(compute_device=torch.device("cpu"), bucket_cap_mb=0)  # unbucketed: one reduce-scatter per unit
    ref = nn.parallel.DistributedDataParallel(Net())
    model = FSDP(Net(lambda m: FSDP(m, **kw)), **kw)
    comm.reset_counters()
    # two accumulation micro-steps then a synchronised one
    with ref.no_sync():
        _loss(ref, _data(rank, 0)).backward()
    _loss(ref, _data(rank, 1)).backward()
    with model.no_sync():
        _loss(model, _data(rank, 0)).backward()
    assert comm.counters()["reduce_scatter"] == 0
    _loss(model, _data(rank, 1)).backward()
    n_inst = len(get_fsdp_instances(model))
    assert comm.counters()["reduce_scatter"] == n_inst, comm.counters()

    with model.summon_full_params():
        names = dict(model.named_parameters())
        ref_params = dict(ref.module.named_parameters())
        # block1/block2 params (not tied) must equal the reference gradient sums after sharding
        assert "block1.0.weight" in names, list(names)
    # gradients: gather shards and compare to DDP's
    flat_ref = torch.cat([p.grad.reshape(-1) for n, p in ref.module.named_parameters() if n.startswith("block1")])
    inst = [m for m in get_fsdp_instances(model) if m is not model][0]
    g = inst.params[0].grad
    gathered = [torch.zeros_like(g) for _ in range(world)]
    dist.all_gather(gathered, g)
    torch.testing.assert_close(torch.cat(gathered)[: flat_ref.numel()], flat_ref, atol=1e-6, rtol=1e-5)

    # summon_full_params writes back local modifications
    with model.summon_full_params():
        with torch.no_grad():
            model.block2[1].bias.fill_(3.0)
    sd = model.state_dict()
    assert torch.all(sd["block2.1.bias"] == 3.0)

    # pickling keeps shards and metadata
    blob = pickle.dumps(model)
    clone = pickle.loads(blob)
    assert clone.process_group == "MISSING"
    for a, b in zip(clone.params, model.params):
        torch.testing.assert_close(a.data, b.data)


def test_fsdp_no_sync_summon_pickle():
    spawn_ranks(_no_sync_and_summon, 2, (), backend="gloo")


def test_fsdp_dummy_group_and_auto_wrap():
    """Construction without torch.distributed, via a dummy group, and size-based auto wrapping."""
    pg = DummyProcessGroup(rank=0, size=1)
    with enable_wrap(wrapper_cls=FSDP, process_group=pg, compute_device=torch.device("cpu")):
        seq = nn.Sequential(nn.Linear(5, 5), nn.Sequential(nn.Linear(5, 5), nn.Linear(5, 5)), nn.Linear(5, 5))
        model = auto_wrap(seq, auto_wrap_policy=functools.partial(default_auto_wrap_policy, min_num_params=40))
        lone = wrap(nn.Linear(3, 3), flatten_parameters=False)
    assert isinstance(model, FSDP)
    assert isinstance(model.module[1], FSDP)
    assert isinstance(model.module[0], nn.Linear)
    assert isinstance(lone, FSDP) and lone.flatten_parameters is False
    out = model(torch.randn(2, 5))
    out.sum().backward()
    assert model.params[0].grad is not None
    assert not isinstance(wrap(nn.Linear(2, 2)), FSDP)  # outside the context
    with pytest.raises(ValueError):
        FSDP(nn.Linear(2, 2), process_group=pg, fp32_reduce_scatter=True)
    with pytest.raises(ValueError):
        FSDP(nn.Linear(2, 2).half(), process_group=pg, mixed_precision=True, compute_device=torch.device("cpu"))
