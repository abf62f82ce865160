"""SlowMo DDP across its settings, on two gloo ranks, each setting against a plain model that is stepped by hand
(the grid of the reference's tests/experimental/nn/data_parallel/test_gossip.py:389-520): slow momentum every step equals
SGD with momentum on the global batch; slow momentum every k steps equals rewinding to the last anchor and taking one
momentum step along the accumulated displacement; LocalSGD every k steps equals averaging the ranks' weights every k
steps.  Then: per-group learning rates in the slow step, a bf16 model with an fp32 master copy, constructor checks, the
communication graphs, uniform mixing, the flatten / communicate helpers and the event recorders."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.experimental.nn.data_parallel import SlowMoBaseAlgorithm, SlowMoDistributedDataParallel
from fairscale_b200.experimental.nn.data_parallel.gossip import (
    DynamicBipartiteExponentialGraph,
    DynamicBipartiteLinearGraph,
    DynamicDirectedExponentialGraph,
    DynamicDirectedLinearGraph,
    NPeerDynamicDirectedExponentialGraph,
    RingGraph,
    UniformMixing,
)
from fairscale_b200.experimental.nn.data_parallel.gossip.utils import cuda_metering, helpers
from fairscale_b200.fair_dev.testing.testing import spawn_ranks

LOCALSGD, SGP = SlowMoBaseAlgorithm.LOCALSGD, SlowMoBaseAlgorithm.SGP


def _net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(2, 10, bias=False), nn.ReLU(), nn.Linear(10, 16), nn.ReLU(), nn.Linear(16, 4, bias=False))


def _step(model, x, y):
    model.train()
    nn.functional.mse_loss(model(x), y).backward()


def _update(opt):
    opt.step()
    opt.zero_grad()


def _pair(rank, world, settings):
    """A plain model and a SlowMo-wrapped copy with the global batch (one sample per rank)."""
    plain, wrapped = _net(), SlowMoDistributedDataParallel(_net(), **settings)
    g = torch.Generator().manual_seed(5)
    return plain, wrapped, torch.randn(world, 2, generator=g), torch.randn(world, 4, generator=g)


def _same(plain, wrapped, atol=1e-6):
    for a, b in zip(plain.parameters(), wrapped.module.parameters()):
        torch.testing.assert_close(b, a, atol=atol, rtol=1e-5)


def _shuffle(x, it):
    return x[torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(1337 + it))]


# ------------------------------------------------------------------------------------------------ slow momentum every step
def _slowmo_every_step(rank, world, settings):
    plain, wrapped, x, y = _pair(rank, world, settings)
    plain_opt = torch.optim.SGD(plain.parameters(), lr=wrapped.slowmo_lr, momentum=wrapped.slowmo_momentum)
    opt = torch.optim.SGD(wrapped.module.parameters(), lr=1, momentum=0)
    wrapped._init_global_momentum_buffers(opt)
    for it in range(3):
        _step(plain, x, y)  # the global batch
        _step(wrapped, x[rank : rank + 1], y[rank : rank + 1])
        _update(plain_opt)
        _update(opt)
        wrapped.perform_slowmo(opt)
        _same(plain, wrapped)
        x = _shuffle(x, it)


@pytest.mark.parametrize("settings", [
    dict(slowmo_base_algorithm=LOCALSGD, localsgd_frequency=1, nprocs_per_node=1, slowmo_momentum=0.0),
    # one node of two processes: gradients are averaged inside the node, nothing is left for LocalSGD to do
    dict(slowmo_base_algorithm=LOCALSGD, localsgd_frequency=100, nprocs_per_node=2, slowmo_momentum=0.0),
    dict(slowmo_base_algorithm=LOCALSGD, localsgd_frequency=1, nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=1, slowmo_memory_efficient=True),
    dict(slowmo_base_algorithm=SGP, nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=1, slowmo_memory_efficient=False),
    dict(slowmo_base_algorithm=LOCALSGD, localsgd_frequency=1, nprocs_per_node=1, slowmo_momentum=0.9, slowmo_lr=0.5, slowmo_frequency=1),
], ids=["localsgd", "two_procs_one_node", "localsgd_slowmo_sharded", "sgp_slowmo", "localsgd_slowmo_lr"])
def test_slow_momentum_every_step_is_momentum_sgd_on_the_global_batch(settings):
    spawn_ranks(_slowmo_every_step, 2, (settings,), backend="gloo")


# ------------------------------------------------------------------------------------------------ slow momentum every k steps
def _slowmo_every_k(rank, world, settings):
    plain, wrapped, x, y = _pair(rank, world, settings)
    plain_opt = torch.optim.SGD(plain.parameters(), lr=1, momentum=0)
    slow_opt = torch.optim.SGD(plain.parameters(), lr=wrapped.slowmo_lr, momentum=wrapped.slowmo_momentum)
    opt = torch.optim.SGD(wrapped.module.parameters(), lr=1, momentum=0)
    wrapped._init_global_momentum_buffers(opt)
    anchor = [p.detach().clone() for p in plain.parameters()]
    for it in range(6):
        _step(plain, x, y)
        _step(wrapped, x[rank : rank + 1], y[rank : rank + 1])
        _update(plain_opt)
        _update(opt)
        wrapped.perform_slowmo(opt)
        if (it + 1) % settings["slowmo_frequency"] == 0:
            # by hand: the displacement since the anchor is the "gradient" of one momentum step taken from the anchor
            with torch.no_grad():
                for p, a in zip(plain.parameters(), anchor):
                    p.grad = a - p
                    p.copy_(a)
            _update(slow_opt)
            with torch.no_grad():
                for p, a in zip(plain.parameters(), anchor):
                    a.copy_(p)
        _same(plain, wrapped, atol=2e-6)
        x = _shuffle(x, it)


@pytest.mark.parametrize("settings", [
    dict(slowmo_base_algorithm=LOCALSGD, localsgd_frequency=1, nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=2, slowmo_memory_efficient=True),
    dict(slowmo_base_algorithm=LOCALSGD, localsgd_frequency=1, nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=2, slowmo_memory_efficient=False),
    dict(slowmo_base_algorithm=SGP, nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=2, slowmo_memory_efficient=True),
    dict(slowmo_base_algorithm=SGP, nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=2, slowmo_memory_efficient=False),
    dict(slowmo_base_algorithm=LOCALSGD, localsgd_frequency=1, nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=2, slowmo_num_shards=1,
         slowmo_memory_efficient=True),
    dict(slowmo_base_algorithm=LOCALSGD, localsgd_frequency=1, nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=3, slowmo_memory_efficient=True),
], ids=["localsgd_sharded", "localsgd_whole", "sgp_sharded", "sgp_whole", "one_shard", "every_third"])
def test_slow_momentum_every_k_steps_rewinds_to_the_anchor(settings):
    spawn_ranks(_slowmo_every_k, 2, (settings,), backend="gloo")


# ------------------------------------------------------------------------------------------------ LocalSGD every k steps
def _localsgd_every_k(rank, world, settings):
    plain, wrapped, x, y = _pair(rank, world, settings)
    assert not wrapped.slowmo
    plain_opt = torch.optim.SGD(plain.parameters(), lr=1, momentum=0)
    opt = torch.optim.SGD(wrapped.module.parameters(), lr=1, momentum=0)
    diverged = False
    for it in range(6):
        for m in (plain, wrapped):
            _step(m, x[rank : rank + 1], y[rank : rank + 1])
        _update(plain_opt)
        _update(opt)
        if (it + 1) % wrapped.localsgd_frequency == 0:
            with torch.no_grad():
                for p in plain.parameters():
                    dist.all_reduce(p)
                    p /= world
        else:
            first = next(plain.parameters()).detach().clone()
            both = [torch.empty_like(first) for _ in range(world)]
            dist.all_gather(both, first)
            diverged = diverged or not torch.equal(both[0], both[1])
        wrapped.perform_slowmo(opt)
        _same(plain, wrapped)
        x = _shuffle(x, it)
    assert diverged  # between two averaging steps the ranks really held different weights


@pytest.mark.parametrize("frequency", [2, 3])
def test_localsgd_every_k_steps_averages_the_weights(frequency):
    settings = dict(slowmo_base_algorithm=LOCALSGD, localsgd_frequency=frequency, nprocs_per_node=1, slowmo_momentum=0.0)
    spawn_ranks(_localsgd_every_k, 2, (settings,), backend="gloo")


# ------------------------------------------------------------------------------------------------ learning rates, master weights
def _two_learning_rates(rank, world):
    """Parameter groups with different learning rates: the slow step divides each parameter's displacement by its own rate."""
    net = _net()
    wrapped = SlowMoDistributedDataParallel(net, nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=1, localsgd_frequency=1)
    groups = [{"params": list(net[0].parameters()), "lr": 0.5}, {"params": list(net[2].parameters()) + list(net[4].parameters()), "lr": 0.1}]
    opt = torch.optim.SGD(groups, lr=0.1)
    wrapped._init_global_momentum_buffers(opt)
    plain = _net()
    plain_groups = [{"params": list(plain[0].parameters()), "lr": 0.5}, {"params": list(plain[2].parameters()) + list(plain[4].parameters()), "lr": 0.1}]
    plain_opt = torch.optim.SGD(plain_groups, lr=0.1, momentum=0.5)  # u = 0.5 u + g; x -= lr u: what slow momentum does with slowmo_lr 1
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(world, 2, generator=g), torch.randn(world, 4, generator=g)
    for it in range(3):
        _step(plain, x, y)
        _step(wrapped, x[rank : rank + 1], y[rank : rank + 1])
        _update(plain_opt)
        _update(opt)
        wrapped.perform_slowmo(opt)
        _same(plain, wrapped, atol=2e-6)


def test_slow_step_uses_each_groups_learning_rate():
    spawn_ranks(_two_learning_rates, 2, (), backend="gloo")


def _master_copy(rank, world, container):
    """bf16 model, fp32 master copy handed to perform_slowmo (flat tensor, list, or one-entry dict): the averaged values land in
    the master copy and the model is refreshed from it; what bf16 cannot carry stays in the master copy (error feedback)."""
    net = nn.Linear(4, 3).bfloat16()
    with torch.no_grad():
        for p in net.parameters():
            p.fill_(float(rank))
    wrapped = SlowMoDistributedDataParallel(net, nprocs_per_node=1, slowmo_momentum=0.0, slowmo_lr=1.0, localsgd_frequency=1)
    masters = [p.detach().float().view(-1).clone() + 0.001 * (rank + 1) for p in net.parameters()]  # below bf16 resolution near 1
    flat = torch.cat(masters)
    arg = {"flat": flat, "list": masters, "dict": {0: flat}}[container]
    before = [m.clone() for m in (masters if container == "list" else [flat])]
    opt = torch.optim.SGD(net.parameters(), lr=0.0)
    wrapped.perform_slowmo(opt, fp32_params=arg)
    after = masters if container == "list" else [flat]
    for a, b in zip(after, before):
        # ranks 0 and 1 averaged: 0.5, plus this rank's own residual (the part of its master copy that was not sent)
        torch.testing.assert_close(a, torch.full_like(a, 0.5 + 0.001 * (rank + 1)), atol=1e-6, rtol=0)
    for p in net.parameters():
        assert torch.equal(p.detach(), torch.full_like(p, 0.5 + 0.001 * (rank + 1)).bfloat16())


@pytest.mark.parametrize("container", ["flat", "list", "dict"])
def test_fp32_master_copy_receives_the_average_and_keeps_its_residual(container):
    spawn_ranks(_master_copy, 2, (container,), backend="gloo")


def _constructor_checks(rank, world):
    with pytest.raises(AssertionError, match="overlap"):
        SlowMoDistributedDataParallel(_net(), nprocs_per_node=1, overlap=True)
    with pytest.raises(AssertionError):
        SlowMoDistributedDataParallel(_net(), nprocs_per_node=0)
    # with momentum 0 and rate 1 the slow step is the identity and is switched off altogether
    plain = SlowMoDistributedDataParallel(_net(), nprocs_per_node=1, slowmo_momentum=0.0, slowmo_lr=1.0)
    assert not plain.slowmo and plain.localsgd and not plain.sgp and plain.comm_device.type == "cpu"
    sharded = SlowMoDistributedDataParallel(_net(), nprocs_per_node=1, slowmo_num_shards=32)
    assert sharded.slowmo_num_shards == world and sharded.is_current_node_a_slowmo_shard
    whole = SlowMoDistributedDataParallel(_net(), nprocs_per_node=1, slowmo_memory_efficient=False)
    assert whole.slowmo_num_shards == 1 and whole.is_current_node_a_slowmo_shard
    one = SlowMoDistributedDataParallel(_net(), nprocs_per_node=1, slowmo_num_shards=1)
    assert one.is_current_node_a_slowmo_shard == (rank == 0)
    # SGP: gossip stops in eval mode and resumes with train(); state dict carries the push-sum weight
    sgp = SlowMoDistributedDataParallel(_net(), nprocs_per_node=1, slowmo_base_algorithm=SGP)
    sgp.eval()
    assert not sgp.gossip_enable and not sgp.training
    sgp.train()
    assert sgp.gossip_enable
    sd = sgp.state_dict()
    assert float(sd["ps_weight"]) == 1.0 and sd["is_sgp_ps_numerator"] is False
    sd["ps_weight"] = torch.tensor([0.25])
    sgp.load_state_dict(sd)
    assert float(sgp.ps_weight) == 0.25
    # buffers follow rank 0 at every forward
    bn = nn.Sequential(nn.Linear(2, 2), nn.BatchNorm1d(2))
    with torch.no_grad():
        bn[1].running_mean.fill_(float(rank + 1))
    ddp = SlowMoDistributedDataParallel(bn, nprocs_per_node=1, slowmo_momentum=0.0)
    ddp.eval()
    ddp(torch.zeros(2, 2))
    assert float(bn[1].running_mean[0]) == 1.0
    dist.barrier()


def test_constructor_checks_flags_and_module_protocol():
    spawn_ranks(_constructor_checks, 2, (), backend="gloo")


# ------------------------------------------------------------------------------------------------ graphs and mixing
GRAPHS = [DynamicDirectedExponentialGraph, NPeerDynamicDirectedExponentialGraph, DynamicBipartiteExponentialGraph,
          DynamicDirectedLinearGraph, DynamicBipartiteLinearGraph, RingGraph]


@pytest.mark.parametrize("cls", GRAPHS)
@pytest.mark.parametrize("world", [2, 4, 8, 16])
def test_every_message_has_a_receiver_that_expects_it(cls, world):
    peers = 2 if cls is RingGraph and world > 2 else 1
    graphs = [cls(r, world, peers_per_itr=peers) for r in range(world)]
    assert len({(g.is_regular_graph(), g.is_bipartite_graph(), g.is_dynamic_graph()) for g in graphs}) == 1
    for _ in range(2 * world):
        views = [g.get_peers(rotate=g.is_dynamic_graph()) for g in graphs]
        for r, (out, inn) in enumerate(views):
            assert len(out) == peers and r not in out
            for dest in out:
                assert r in views[dest][1], (cls.__name__, world, r, dest)
            for src in inn:
                assert r in views[src][0]
        if graphs[0].is_regular_graph():
            assert all(len(out) == len(inn) for out, inn in views)
    if graphs[0].is_bipartite_graph():
        assert [g.is_passive() for g in graphs] == [r % 2 == 0 for r in range(world)]
        assert graphs[0].is_passive(1) is False
    else:
        assert not any(g.is_passive() for g in graphs)


@pytest.mark.parametrize("cls,steps", [(NPeerDynamicDirectedExponentialGraph, 4), (DynamicDirectedExponentialGraph, 7)])
def test_exponential_graphs_reach_everybody_in_one_cycle(cls, steps):
    """Forward hops 1, 2, 4, 8 spread a value over 16 ranks in log2(16) pushes; the graph that also hops backwards has seven
    distinct peers per rank and needs one cycle through them at most."""
    world = 16
    graphs = [cls(r, world) for r in range(world)]
    knows = [{r} for r in range(world)]
    for _ in range(steps):
        views = [g.get_peers(rotate=True) for g in graphs]
        new = [set(k) for k in knows]
        for r, (out, _) in enumerate(views):
            for dest in out:
                new[dest] |= knows[r]
        knows = new
    assert all(len(k) == world for k in knows)


def test_peers_per_iteration_can_be_changed_and_nodes_map_to_process_ranks():
    g = NPeerDynamicDirectedExponentialGraph(0, 9, peers_per_itr=2)
    out, _ = g.get_peers()
    assert len(out) == 2
    g.peers_per_itr = 1
    assert g.peers_per_itr == 1 and len(g.get_peers()[0]) == 1
    with pytest.raises(AssertionError):
        RingGraph(0, 4, peers_per_itr=0)
    # two processes per node: edges connect the nodes' first processes
    g = DynamicDirectedExponentialGraph(1, 4, nprocs_per_node=2)
    out_edges, in_edges = g.get_edges()
    assert all(e.dest % 2 == 0 and e.src == 2 for e in out_edges) and all(e.dest == 2 for e in in_edges)
    assert "->" in repr(out_edges[0])


def test_uniform_mixing_weights():
    g = RingGraph(0, 6, peers_per_itr=2)
    mixing = UniformMixing(g, torch.device("cpu"))
    assert mixing.is_uniform() and mixing.is_regular()
    w = mixing.get_mixing_weights(residual_adjusted=False)
    out, _ = g.get_peers()
    assert set(w) == {"lo", "uniform", *out}
    total = float(w["lo"]) + sum(float(w[p]) for p in out)
    assert abs(total - 1.0) < 1e-6 and abs(float(w["lo"]) - 1 / 3) < 1e-6
    adjusted = mixing.get_mixing_weights(residual_adjusted=True)
    assert float(adjusted["lo"]) == float(w["lo"]) and all(float(adjusted[p]) == 1.0 for p in out)


# ------------------------------------------------------------------------------------------------ helpers
def test_flatten_unflatten_group_and_communicate():
    a, b, c = torch.arange(6.0).view(2, 3), torch.ones(4, dtype=torch.float64), torch.full((2,), 7.0)
    flat = helpers.flatten_tensors([a, c])
    assert flat.tolist() == [0, 1, 2, 3, 4, 5, 7, 7]
    flat[0] = 100.0
    assert float(a[0, 0]) == 0.0  # a copy, also for a single tensor
    assert helpers.flatten_tensors([a]).data_ptr() != a.data_ptr()
    back = helpers.unflatten_tensors(flat, [a, c])
    assert back[0].shape == a.shape and back[1].shape == c.shape and back[0].data_ptr() == flat.data_ptr()
    groups = helpers.group_by_dtype([a, b, c])
    assert list(groups) == [torch.float32, torch.float64] and len(groups[torch.float32]) == 2

    calls = []

    def double(tensor):
        calls.append((tensor.dtype, tensor.numel()))
        tensor.mul_(2)

    helpers.communicate([a, b, c], double)
    assert calls == [(torch.float32, 8), (torch.float64, 4)]  # once per dtype, on the flattened group
    assert float(a[1, 2]) == 10.0 and float(b[0]) == 2.0 and float(c[0]) == 14.0

    log = helpers.make_logger(3, verbose=False)
    assert helpers.make_logger(3) is log and len(log.handlers) == 1
    adapter = helpers.MultiProcessAdapter(log, {"process_num": 3})
    assert adapter.process("hello", {})[0] == "process: 3 hello"


def test_event_recorders_without_a_gpu():
    rec = cuda_metering.create_event_recorder("phase", dummy=True)
    assert isinstance(rec, cuda_metering.DummyCudaEventRecorder)
    rec.stop()  # nothing to record, nothing to fail
    cuda_metering.CudaEventRecorder.reset()
    assert "phase" not in cuda_metering.CudaEventRecorder.get_timings()
    assert len(cuda_metering.deque_with_max_len_fixed()) == 0 and cuda_metering.deque_with_max_len_fixed().maxlen is not None


def _profile_mode(rank, world):
    # profile mode asks for event recorders; on a machine without CUDA they fall back to the dummies and training still runs
    wrapped = SlowMoDistributedDataParallel(_net(), nprocs_per_node=1, profile_mode=torch.cuda.is_available(), verbose=True)
    opt = torch.optim.SGD(wrapped.module.parameters(), lr=0.1)
    _step(wrapped, torch.randn(1, 2), torch.randn(1, 4))
    _update(opt)
    wrapped.perform_slowmo(opt)
    assert wrapped.num_updates == 1
    frozen = copy.deepcopy(wrapped.module.state_dict())
    wrapped.load_state_dict(wrapped.state_dict())
    assert all(torch.equal(v, frozen[k]) for k, v in wrapped.module.state_dict().items())


def test_verbose_wrapper_trains_and_round_trips_its_state_dict():
    spawn_ranks(_profile_mode, 2, (), backend="gloo")
