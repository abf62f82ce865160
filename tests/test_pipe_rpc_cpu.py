"""PipeRPCWrapper: rank 0 drives a two-stage pipeline on two RPC workers; the loss is computed on rank 0 although the
last stage lives on the other worker, and ``loss.backward()`` alone runs every stage's backward."""
import torch
from torch import nn

from fairscale_b200.fair_dev.testing.testing import find_free_port, spawn_ranks


def _factory():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(6, 6), nn.Tanh(), nn.Linear(6, 3))


def _stage_grads(pipe):
    return [p.grad.clone() for p in pipe.parameters()]


def _worker(rank, world, port):
    from torch.distributed import rpc

    from fairscale_b200.nn.pipe import PipeRPCWrapper

    rpc.init_rpc(f"Test{rank}", rank=rank, world_size=world,
                 rpc_backend_options=rpc.TensorPipeRpcBackendOptions(init_method=f"tcp://127.0.0.1:{port}", _transports=["uv"]))
    try:
        if rank == 0:
            wrapper = PipeRPCWrapper(_factory, [2, 1], chunks=2, checkpoint="never")
            oracle = _factory()
            x = torch.randn(4, 6)
            out = wrapper(x)
            ref = oracle(x)
            torch.testing.assert_close(out, ref, atol=1e-6, rtol=1e-5)
            out.pow(2).sum().backward()
            ref.pow(2).sum().backward()
            mine = _stage_grads(wrapper.model)
            torch.testing.assert_close(mine[0], oracle[0].weight.grad, atol=1e-5, rtol=1e-5)
            theirs = wrapper.foreach_worker(_stage_grads)[0]
            torch.testing.assert_close(theirs[0], oracle[2].weight.grad, atol=1e-5, rtol=1e-5)
            # evaluation: no graph, nothing to redirect
            wrapper.eval()
            with torch.no_grad():
                assert not wrapper(x).requires_grad
    finally:
        rpc.shutdown()


def test_pipe_rpc_wrapper_loss_on_rank0():
    spawn_ranks(_worker, 2, (find_free_port(),), backend="gloo")
