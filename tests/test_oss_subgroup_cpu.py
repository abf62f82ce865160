"""OSS and ShardedDataParallel in a process group whose members are not the first ranks of the world and not consecutive
(the case of the reference's tests/optim/test_oss.py::test_multiple_groups, which catches local ranks used where global ones
are needed): ranks 1 and 3 of four train together, the others stand by."""
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.data_parallel import ShardedDataParallel
from fairscale_b200.optim import OSS

MEMBERS = [1, 3]


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(6, 12), nn.Tanh(), nn.Linear(12, 12), nn.Tanh(), nn.Linear(12, 3))


def _in_sync(model, group):
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    everyone = [torch.empty_like(flat) for _ in MEMBERS]
    dist.all_gather(everyone, flat, group=group)
    return all(torch.equal(everyone[0], e) for e in everyone)


def _worker(rank, world, wrap_with_sdp):
    group = dist.new_group(ranks=MEMBERS)  # every rank of the world takes part in creating it
    if rank not in MEMBERS:
        dist.barrier()
        return
    torch.manual_seed(rank)  # different data per member
    model = _model()
    oss = OSS(model.parameters(), optim=torch.optim.SGD, group=group, lr=0.1, momentum=0.9)
    assert oss.world_size == 2 and oss.rank == MEMBERS.index(rank)
    owned = sum(p.numel() for g in oss.optim.param_groups for p in g["params"])
    assert 0 < owned < sum(p.numel() for p in model.parameters())
    sdp = ShardedDataParallel(model, oss, process_group=group) if wrap_with_sdp else None
    ref = _model()
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    for step in range(4):
        x, y = torch.randn(5, 6), torch.randn(5, 3)
        oss.zero_grad()
        loss = nn.functional.mse_loss((sdp or model)(x), y)
        loss.backward()
        if sdp is None:  # reduce by hand: average over the group
            for p in model.parameters():
                dist.all_reduce(p.grad, group=group)
                p.grad /= 2
        oss.step()
        assert _in_sync(model, group), f"replicas drifted apart at step {step}"
        # the same update by hand on a plain copy
        ref_opt.zero_grad()
        nn.functional.mse_loss(ref(x), y).backward()
        for p in ref.parameters():
            dist.all_reduce(p.grad, group=group)
            p.grad /= 2
        ref_opt.step()
    for a, b in zip(model.parameters(), ref.parameters()):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)
    # consolidation names the recipient by its rank in the group; the state comes back complete
    oss.consolidate_state_dict(recipient_rank=1)
    if oss.rank == 1:
        state = oss.state_dict()
        assert len(state["state"]) == len(list(model.parameters()))
    # (clip_grad_norm is not called here: like the reference it sums the norm over the whole world, so that model-parallel
    # ranks outside the optimizer's group are counted, which needs every rank of the world to call it)
    dist.barrier()


def test_oss_in_a_group_of_non_consecutive_ranks():
    spawn_ranks(_worker, 4, (False,), backend="gloo")


def test_sharded_ddp_in_a_group_of_non_consecutive_ranks():
    spawn_ranks(_worker, 4, (True,), backend="gloo")
