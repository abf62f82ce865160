"""SlowMo DDP on gloo ranks: LocalSGD averaging, slow momentum vs a closed-form oracle, SGP consensus."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.experimental.nn.data_parallel import SlowMoBaseAlgorithm, SlowMoDistributedDataParallel
from fairscale_b200.experimental.nn.data_parallel.gossip import DynamicDirectedExponentialGraph, RingGraph
from fairscale_b200.fair_dev.testing.testing import spawn_ranks


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(4, 6), nn.Tanh(), nn.Linear(6, 2))


def _localsgd_slowmo(rank, world, mem_eff):
    model = SlowMoDistributedDataParallel(_model(), nprocs_per_node=1, slowmo_momentum=0.5, slowmo_frequency=2, localsgd_frequency=1,
                                          slowmo_memory_efficient=mem_eff, slowmo_num_shards=2)
    opt = torch.optim.SGD(model.module.parameters(), lr=0.1)
    model._init_global_momentum_buffers(opt)  # anchor the slow weights at the common initial point
    # oracle: every rank simulates all ranks
    replicas = [_model() for _ in range(world)]
    opts = [torch.optim.SGD(m.parameters(), lr=0.1) for m in replicas]
    old = torch.cat([p.detach().reshape(-1) for p in replicas[0].parameters()])
    u = torch.zeros_like(old)
    for step in range(4):
        for r in range(world):
            torch.manual_seed(100 * step + r)
            x = torch.randn(3, 4)
            opts[r].zero_grad()
            replicas[r](x).pow(2).sum().backward()
            opts[r].step()
            if r == rank:
                opt.zero_grad()
                model(x).pow(2).sum().backward()
                opt.step()
        model.perform_slowmo(opt)
        with torch.no_grad():
            avg = [torch.stack([list(m.parameters())[i] for m in replicas]).mean(0) for i in range(4)]
            if (step + 1) % 2 == 0:
                flat = torch.cat([a.reshape(-1) for a in avg])
                u = 0.5 * u + (old - flat) / 0.1
                old = old - 0.1 * u
                off = 0
                for i, a in enumerate(avg):
                    avg[i] = old[off : off + a.numel()].view_as(a)
                    off += a.numel()
            for m in replicas:
                for p, a in zip(m.parameters(), avg):
                    p.copy_(a)
        for p, q in zip(model.module.parameters(), replicas[0].parameters()):
            torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("mem_eff", [True, False])
def test_localsgd_with_slow_momentum_matches_oracle(mem_eff):
    spawn_ranks(_localsgd_slowmo, 2, (mem_eff,), backend="gloo")


def _sgp(rank, world, ring):
    m = nn.Linear(3, 1, bias=False)
    with torch.no_grad():
        m.weight.fill_(float(rank))
    graph = RingGraph(rank, world, peers_per_itr=2) if ring else None
    model = SlowMoDistributedDataParallel(m, nprocs_per_node=1, slowmo_base_algorithm=SlowMoBaseAlgorithm.SGP, slowmo_momentum=0.0,
                                          slowmo_lr=1.0, graph=graph)
    opt = torch.optim.SGD(m.parameters(), lr=0.0)
    total = torch.zeros(1)
    for _ in range(12):
        model.perform_slowmo(opt)
        s = m.weight.detach().sum().reshape(1) / 3
        dist.all_reduce(s)
        torch.testing.assert_close(s, torch.tensor([float(sum(range(world)))]))  # gossip conserves the mean
    torch.testing.assert_close(m.weight.detach(), torch.full((1, 3), (world - 1) / 2.0), rtol=0, atol=1e-2)
    sd = model.state_dict()
    assert "ps_weight" in sd
    model.load_state_dict(sd)


@pytest.mark.parametrize("ring", [False, True])
def test_sgp_reaches_consensus(ring):
    spawn_ranks(_sgp, 4, (ring,), backend="gloo")


def _two_per_node(rank, world):
    model = SlowMoDistributedDataParallel(_model(), nprocs_per_node=2, slowmo_momentum=0.0, slowmo_lr=1.0, localsgd_frequency=1)
    opt = torch.optim.SGD(model.module.parameters(), lr=0.1)
    torch.manual_seed(rank)
    model(torch.randn(3, 4)).pow(2).sum().backward()
    g = [p.grad.clone() for p in model.module.parameters()]
    peer = [torch.zeros_like(x) for x in g]
    # gradients were averaged inside the node: both ranks of a node hold the same gradient
    for a in g:
        both = [torch.zeros_like(a) for _ in range(world)]
        dist.all_gather(both, a)
        node = rank // 2
        torch.testing.assert_close(both[2 * node], both[2 * node + 1])
    opt.step()
    model.perform_slowmo(opt)
    for p in model.module.parameters():
        allp = [torch.zeros_like(p) for _ in range(world)]
        dist.all_gather(allp, p.detach())
        for q in allp[1:]:
            torch.testing.assert_close(allp[0], q)


def test_two_procs_per_node_groups():
    spawn_ranks(_two_per_node, 4, (), backend="gloo")


def test_graphs_are_consistent():
    for cls in (DynamicDirectedExponentialGraph, RingGraph):
        graphs = [cls(r, 8, peers_per_itr=1) for r in range(8)]
        for _ in range(4):
            outs = [g.get_peers(rotate=g.is_dynamic_graph()) for g in graphs]
            for r, (o, i) in enumerate(outs):
                for dest in o:
                    assert r in outs[dest][1]
