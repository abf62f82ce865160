"""The pipe's checkpoint (Checkpoint / Recompute pair) used as a plain checkpoint function under DistributedDataParallel
on gloo ranks (cases of the reference's tests/nn/pipe/test_checkpoint_ddp.py): the whole model, two layers sharing a weight,
only the second half of a model - gradients equal those without checkpointing and those of torch.utils.checkpoint."""
import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.nn.parallel import DistributedDataParallel as DDP
from torch.utils.checkpoint import checkpoint as torch_checkpoint

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.pipe.checkpoint import Checkpointing
from fairscale_b200.nn.pipe.microbatch import Batch


def pipe_checkpoint(function, input):
    """The pipe's two-node checkpoint behind the interface of ``torch.utils.checkpoint.checkpoint``."""
    batch = Batch(input, 0)
    chk = Checkpointing(function, batch)
    batch = chk.checkpoint()
    chk.recompute(batch)
    return batch.tensor_or_tensors


def _plain(function, input):
    return function(input)


def _torch(function, input):
    return torch_checkpoint(function, input, use_reentrant=True)


class _Half(nn.Module):
    def __init__(self, checkpoint):
        super().__init__()
        self.l1, self.l2 = nn.Linear(64, 64), nn.Linear(64, 64)
        self.checkpoint = checkpoint

    def forward(self, x):
        return self.checkpoint(self.l2, self.l1(x))


def _grads(rank, case, checkpoint):
    torch.manual_seed(31415)
    if case == "whole":
        model = nn.Sequential(nn.Linear(64, 64), nn.Linear(64, 64))
    elif case == "shared":
        l1, l2 = nn.Linear(64, 64), nn.Linear(64, 64)
        l1.weight = l2.weight
        model = nn.Sequential(l1, l2)
    else:
        model = _Half(checkpoint)
    ddp = DDP(model)
    x = torch.rand(16, 64, generator=torch.Generator().manual_seed(rank)).requires_grad_()
    out = ddp(x) if case == "half" else checkpoint(ddp, x)
    assert all(p.grad is None for p in model.parameters())
    out.sum().backward()
    return [p.grad.clone() for p in model.parameters()], x.grad.clone()


def _worker(rank, world, case):
    want, want_x = _grads(rank, case, _plain)
    for checkpoint in (pipe_checkpoint, _torch):
        got, got_x = _grads(rank, case, checkpoint)
        assert len(got) == len(want)
        for a, b in zip(got, want):
            torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)
        torch.testing.assert_close(got_x, want_x, atol=1e-6, rtol=1e-5)
    # the gradients are the averages over the ranks: every rank holds the same ones
    flat = torch.cat([g.reshape(-1) for g in want])
    both = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(both, flat)
    assert torch.equal(both[0], both[1])


@pytest.mark.parametrize("case", ["whole", "shared", "half"])
def test_pipe_checkpoint_under_ddp(case):
    spawn_ranks(_worker, 2, (case,), backend="gloo")
