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


def _static_worker(rank, world):
    """Three steps with fixed shapes: with the static contract only the first step's messages carry a header."""
    pipe = AsyncPipe(nn.Sequential(*_layers()), balance=[2, 2, 1], chunks=3, checkpoint="never")
    pipe.transport.static_shapes = True
    torch.manual_seed(5)
    x = torch.randn(6, 6)
    counts, posted_ahead = [], []
    for _ in range(3):
        out = pipe(x if rank == 0 else None)
        if rank == 2:
            out.sum().backward()
            pipe.back_helper()
        elif rank < 2:
            pipe.back_helper(out)
        counts.append((pipe.transport.headers_sent, pipe.transport.headers_received))
        posted_ahead.append(pipe.transport.prefetches)
        dist.barrier()
    if rank < 3:
        assert counts[1] != counts[0] or rank == 3  # the chunk-count message has no slot and keeps its header
        per_step_after_first = (counts[2][0] - counts[1][0], counts[2][1] - counts[1][1])
        first_step = counts[0]
        assert per_step_after_first[0] < first_step[0] or first_step[0] == 0
        assert per_step_after_first[1] < first_step[1] or first_step[1] == 0
        assert per_step_after_first[0] <= 1 and per_step_after_first[1] <= 1  # only the chunk-count message
    # once the shapes are known, receives are posted one message ahead: activations on every stage but the first, gradients
    # on every stage but the last (chunks - 1 of each per step)
    if rank in (1, 2):
        assert posted_ahead[0] == 0 and posted_ahead[2] > posted_ahead[1] > 0, posted_ahead
    if rank == 1:
        # a tensor that breaks the contract is refused by the sender
        with pytest.raises(RuntimeError, match="static contract"):
            pipe.transport.send(torch.zeros(5, 5), 2, slot=0)
    dist.barrier()


def test_static_shape_contract_skips_headers_after_the_first_step():
    spawn_ranks(_static_worker, 4, (), backend="gloo")
