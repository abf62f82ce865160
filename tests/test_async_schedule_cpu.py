"""Event-loop schedule of the multi-process pipeline: a layer that is called twice makes the data revisit its stage."""
import copy

import pytest
import torch
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.pipe import AsyncPipe
from fairscale_b200.nn.pipe.async_pipe import plan_invocations
from fairscale_b200.nn.pipe.async_schedule import AutogradWithoutActivations, Location


def test_plan_invocations_maps_shared_layers_to_their_first_stage():
    a, b, c = nn.Linear(2, 2), nn.Linear(2, 2), nn.Linear(2, 2)
    locations, invocations = plan_invocations([a, b, a, c], [2, 2])
    assert locations == [Location(0, 0), Location(0, 1), Location(0, 0), Location(1, 0)]
    assert [inv.order for inv in invocations] == [0, 1, 2, 3]
    assert invocations[0].source is None and invocations[3].dest is None
    assert invocations[2].source == Location(0, 1) and invocations[2].dest == Location(1, 0)


def test_autograd_without_activations_feeds_the_attached_gradient():
    x = torch.randn(3, 4, requires_grad=True)
    y = x * 2
    stand_in = AutogradWithoutActivations.apply(y)
    assert stand_in.shape == (1,)
    stand_in.grad_fn.grad_from_pipeline = (torch.ones(3, 4),)
    stand_in.backward(torch.ones(1))
    assert torch.equal(x.grad, torch.full((3, 4), 2.0))


def _worker(rank, world, checkpoint, balance):
    torch.manual_seed(0)
    a, b, c = nn.Linear(8, 8), nn.Linear(8, 8), nn.Linear(8, 4)
    seq = nn.Sequential(a, nn.Tanh(), b, nn.Tanh(), a, c)  # `a` runs twice: stage 0 -> 1 -> 0 -> 1
    oracle = copy.deepcopy(seq)
    pipe = AsyncPipe(seq, balance, chunks=3, checkpoint=checkpoint)
    x = torch.randn(6, 8)
    for _ in range(2):  # two steps: the loop state is rebuilt every mini-batch
        pipe.zero_grad()
        oracle.zero_grad()
        out = pipe(x if rank == 0 else None)
        tail = len(balance) - 1
        ref = oracle(x)
        ref.pow(2).sum().backward()
        if rank == tail:
            torch.testing.assert_close(out, ref, atol=1e-6, rtol=1e-5)
            out.pow(2).sum().backward()
        else:
            assert out is None
        pipe.back_helper()
        owned = {0: [(a, oracle[0])], tail: [(c, oracle[5])]}
        owned.setdefault(1, []).append((b, oracle[2]))
        for mine, theirs in owned.get(rank, []):
            if rank < len(balance):
                torch.testing.assert_close(mine.weight.grad, theirs.weight.grad, atol=1e-5, rtol=1e-5)
                torch.testing.assert_close(mine.bias.grad, theirs.bias.grad, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("checkpoint", ["never", "always"])
def test_shared_layer_across_two_stages(checkpoint):
    spawn_ranks(_worker, 2, (checkpoint, [2, 4]), backend="gloo")


def test_shared_layer_three_stages():
    spawn_ranks(_worker, 3, ("except_last", [2, 2, 2]), backend="gloo")


def _rpc_worker(rank, world, port):
    import os

    from torch.distributed import rpc

    from fairscale_b200.nn.pipe.messages import RpcTransport

    rpc.init_rpc(f"Test{rank}", rank=rank, world_size=world,
                 rpc_backend_options=rpc.TensorPipeRpcBackendOptions(init_method=f"tcp://127.0.0.1:{port}", _transports=["uv"]))
    os.environ["FORCE_RPC"] = "1"
    try:
        torch.manual_seed(0)
        seq = nn.Sequential(nn.Linear(8, 8), nn.Tanh(), nn.Linear(8, 4))
        oracle = copy.deepcopy(seq)
        pipe = AsyncPipe(seq, [2, 1], chunks=2, checkpoint="never")
        assert isinstance(pipe.transport, RpcTransport)
        x = torch.randn(4, 8)
        out = pipe(x if rank == 0 else None)
        ref = oracle(x)
        ref.sum().backward()
        if rank == 1:
            torch.testing.assert_close(out, ref, atol=1e-6, rtol=1e-5)
            out.sum().backward()
            torch.testing.assert_close(seq[2].weight.grad, oracle[2].weight.grad, atol=1e-5, rtol=1e-5)
        pipe.back_helper(out if rank == 0 else None)
        if rank == 0:
            torch.testing.assert_close(seq[0].weight.grad, oracle[0].weight.grad, atol=1e-5, rtol=1e-5)
    finally:
        os.environ.pop("FORCE_RPC", None)
        rpc.shutdown()


def test_async_pipe_over_rpc_transport():
    from fairscale_b200.fair_dev.testing.testing import find_free_port

    spawn_ranks(_rpc_worker, 2, (find_free_port(),), backend="gloo")
