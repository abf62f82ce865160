"""Multi-process pipeline over gloo p2p: output and gradients equal the single-process model."""
import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.pipe import AsyncPipe, LazyModule


def _layers():
    torch.manual_seed(0)
    return [nn.Linear(6, 12), nn.Tanh(), nn.Linear(12, 12), nn.ReLU(), nn.Linear(12, 3)]


def _worker(rank, world, checkpoint, lazy):
    ref = nn.Sequential(*_layers())
    if lazy:
        made = _layers()
        module = [LazyModule(lambda m=m: m) for m in made]
    else:
        module = nn.Sequential(*_layers())
    pipe = AsyncPipe(module, balance=[2, 2, 1], chunks=3, checkpoint=checkpoint)
    torch.manual_seed(5)
    x = torch.randn(6, 6)
    out = pipe(x if rank == 0 else None)
    if rank == 2:
        y_ref = ref(x)
        torch.testing.assert_close(out, y_ref)
        out.pow(2).sum().backward()
        pipe.back_helper()
    elif rank < 2:
        pipe.back_helper(out)
    ref_out = ref(x)
    ref_out.pow(2).sum().backward()
    if rank < 3:
        lo = sum([2, 2, 1][:rank])
        ref_params = [p for l in list(ref)[lo : lo + [2, 2, 1][rank]] for p in l.parameters()]
        for a, b in zip(pipe.partition.parameters(), ref_params):
            torch.testing.assert_close(a.grad, b.grad, atol=1e-6, rtol=1e-5)
    else:
        assert pipe.partition is None
    dist.barrier()


@pytest.mark.parametrize("checkpoint,lazy", [("never", False), ("always", True), ("except_last", False)])
def test_async_pipe_matches_sequential(checkpoint, lazy):
    spawn_ranks(_worker, 4, (checkpoint, lazy), backend="gloo")
