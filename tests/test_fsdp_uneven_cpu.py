"""FSDP with more ranks than some parameters have elements, and full state carried between world sizes (gloo, CPU)."""
import copy

import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn import FullyShardedDataParallel as FSDP


def _tiny():
    torch.manual_seed(3)
    # the 1-element and 2-element parameters are smaller than the world: most ranks hold only padding for them
    return nn.Sequential(nn.Linear(3, 1, bias=True), nn.Linear(1, 2, bias=False), nn.Linear(2, 5))


def _batch(rank, step):
    g = torch.Generator().manual_seed(50 * step + rank)
    return torch.randn(6, 3, generator=g)


def _run(model, opt, rank, steps):
    losses = []
    for s in range(steps):
        opt.zero_grad()
        loss = model(_batch(rank, s)).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses


def _uneven(rank, world, flatten):
    ref = nn.parallel.DistributedDataParallel(_tiny())
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    kw = dict(compute_device=torch.device("cpu"), flatten_parameters=flatten)
    layers = list(_tiny())
    model = FSDP(nn.Sequential(FSDP(layers[0], **kw), FSDP(layers[1], **kw), layers[2]), **kw)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    torch.testing.assert_close(torch.tensor(_run(model, opt, rank, 3)), torch.tensor(_run(ref, ref_opt, rank, 3)), atol=1e-6, rtol=1e-5)
    full = model.state_dict()
    for k, v in ref.module.state_dict().items():
        torch.testing.assert_close(full[k], v, atol=1e-6, rtol=1e-5)
    # every rank holds a shard of the same (padded) length
    for p in model.params:
        sizes = [torch.zeros(1, dtype=torch.long) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([p.numel()]))
        assert len({int(s) for s in sizes}) == 1


def test_fsdp_three_ranks_tiny_params_flat():
    spawn_ranks(_uneven, 3, (True,), backend="gloo")


def test_fsdp_three_ranks_tiny_params_unflat():
    spawn_ranks(_uneven, 3, (False,), backend="gloo")


def _save(rank, world, path):
    kw = dict(compute_device=torch.device("cpu"))
    model = FSDP(_tiny(), **kw)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    _run(model, opt, rank, 2)
    weights = model.state_dict()
    osd = model.gather_full_optim_state_dict(opt)
    if rank == 0:
        torch.save({"weights": weights, "optim": osd}, path)


def _resume(rank, world, path):
    ckpt = torch.load(path, weights_only=False)
    kw = dict(compute_device=torch.device("cpu"))
    model = FSDP(_tiny(), **kw)
    model.load_state_dict(ckpt["weights"])
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    opt.load_state_dict(model.get_shard_from_optim_state_dict(copy.deepcopy(ckpt["optim"])))
    # the re-sharded Adam moments, gathered again, are the saved ones
    again = model.gather_full_optim_state_dict(opt)
    if rank == 0:
        for pid, st in ckpt["optim"]["state"].items():
            torch.testing.assert_close(again["state"][pid]["exp_avg"], st["exp_avg"])
            torch.testing.assert_close(again["state"][pid]["exp_avg_sq"], st["exp_avg_sq"])
    full = model.state_dict()
    for k, v in ckpt["weights"].items():
        torch.testing.assert_close(full[k], v)
    _run(model, opt, rank, 1)  # and training goes on


def test_fsdp_checkpoint_moves_between_world_sizes(tmp_path):
    path = str(tmp_path / "ckpt.pt")
    spawn_ranks(_save, 2, (path,), backend="gloo")
    spawn_ranks(_resume, 3, (path,), backend="gloo")
