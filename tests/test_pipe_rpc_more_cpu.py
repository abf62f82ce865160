"""PipeRPCWrapper on three RPC workers (cases of the reference's tests/nn/pipe_process/test_rpc.py): every worker registers an
optimizer for its stage through ``foreach_worker``, one training step is driven from rank 0 and compared with the same model
trained in one process, then both are evaluated; with a plain chain of layers and with one layer object used by three
stages."""
import copy

import pytest
import torch
from torch import nn

from fairscale_b200.fair_dev.testing.testing import find_free_port, spawn_ranks


def _chain():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(10, 10), nn.ReLU(), nn.Linear(10, 10), nn.ReLU(), nn.Linear(10, 10), nn.ReLU())


def _reused():
    torch.manual_seed(0)
    shared = nn.Linear(10, 10)
    return [shared, nn.ReLU(), shared, nn.Tanh(), shared, nn.Sigmoid()]


def _register_optimizer(pipe):
    params = list(pipe.parameters())
    pipe.optimizer = torch.optim.SGD(params, lr=0.01, momentum=0.9) if params else None
    return len(params)


def _step_optimizer(pipe):
    if pipe.optimizer is not None:
        pipe.optimizer.step()
        pipe.optimizer.zero_grad()
    return True


def _check(factory, balance, checkpoint):
    from fairscale_b200.nn.pipe import PipeRPCWrapper

    made = factory()
    oracle = nn.Sequential(*made) if isinstance(made, list) else made
    oracle = copy.deepcopy(oracle)
    wrapper = PipeRPCWrapper(factory, balance, chunks=2, checkpoint=checkpoint)
    counts = wrapper.foreach_worker(_register_optimizer, include_self=True)
    assert sum(counts) == len({id(p) for p in oracle.parameters()}) and len(counts) == 3
    oracle_opt = torch.optim.SGD(oracle.parameters(), lr=0.01, momentum=0.9)

    g = torch.Generator().manual_seed(1)
    x, target = torch.rand(4, 10, generator=g), torch.rand(4, 10, generator=g)
    for _ in range(2):
        out, ref = wrapper(x), oracle(x)
        torch.testing.assert_close(out, ref, atol=1e-6, rtol=1e-5)
        nn.functional.mse_loss(out, target).backward()   # runs the backward of every worker
        nn.functional.mse_loss(ref, target).backward()
        assert all(wrapper.foreach_worker(_step_optimizer, include_self=True))
        oracle_opt.step()
        oracle_opt.zero_grad()
    wrapper.eval()
    oracle.eval()
    with torch.no_grad():
        torch.testing.assert_close(wrapper(x), oracle(x), atol=1e-6, rtol=1e-5)
    assert wrapper.final_stage == len(balance) - 1


def _worker(rank, world, port, case):
    from torch.distributed import rpc

    import fairscale_b200.nn.pipe  # noqa: F401  (imported before the agent's threads could race to do it)

    rpc.init_rpc(f"Test{rank}", rank=rank, world_size=world,
                 rpc_backend_options=rpc.TensorPipeRpcBackendOptions(init_method=f"tcp://127.0.0.1:{port}", _transports=["uv"]))
    try:
        if rank == 0:
            if case == "chain":
                for mode in ("except_last", "never", "always"):
                    _check(_chain, [2, 2, 2], mode)
            else:
                _check(_reused, [2, 2, 2], "never")
    finally:
        rpc.shutdown()


@pytest.mark.parametrize("case", ["chain", "reused_layer"])
def test_training_step_driven_from_rank_zero(case):
    spawn_ranks(_worker, 3, (find_free_port(), case), backend="gloo")
