"""RPC pipeline on two CPU workers: forward equals the local model; distributed autograd + optimizer train it."""
import os

import pytest
import torch
from torch import nn

from fairscale_b200.fair_dev.testing.testing import find_free_port, spawn_ranks


def _run(rank, world, port, mode):
    import torch.distributed.autograd as dist_autograd
    from torch.distributed import rpc
    from torch.distributed.nn import RemoteModule
    from torch.distributed.optim import DistributedOptimizer

    from fairscale_b200.experimental.nn.distributed_pipeline import DistributedLoss, DistributedPipeline, PipelineModulesGraph, make_graph

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    rpc.init_rpc(f"worker{rank}", rank=rank, world_size=world,
                 rpc_backend_options=rpc.TensorPipeRpcBackendOptions(init_method=f"tcp://127.0.0.1:{port}", _transports=["uv"]))
    if rank == 0:
        torch.manual_seed(0)
        l1 = RemoteModule("worker0/cpu", nn.Linear, (4, 8))
        act = RemoteModule("worker0/cpu", nn.ReLU, ())
        l2 = RemoteModule("worker1/cpu", nn.Linear, (8, 8))
        l3 = RemoteModule("worker1/cpu", nn.Linear, (8, 2))
        if mode == "graph":
            g = PipelineModulesGraph()
            g.add_sequence([l1, act, l2, l3], [0])
        else:
            class M(nn.Module):
                def __init__(self):
                    super().__init__()
                    self.l1, self.act, self.l2, self.l3 = l1, act, l2, l3

                def forward(self, x):
                    return self.l3(self.l2(self.act(self.l1(x))))

            g = make_graph(M())
        pipe = DistributedPipeline(g, chunks=2, checkpoint="except_last")
        assert len(pipe.partitions) == 2
        x = torch.randn(6, 4)
        y = pipe(x).to_here()
        local = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 8), nn.Linear(8, 2))
        for dst, src in zip(local.parameters(), [r.to_here() for r in pipe.parameter_rrefs()]):
            dst.data.copy_(src)
        torch.testing.assert_close(y, local(x))
        opt = DistributedOptimizer(torch.optim.SGD, pipe.parameter_rrefs(), lr=0.05)
        loss_fn = DistributedLoss(nn.MSELoss)
        target = torch.zeros(6, 2)
        losses = []
        for _ in range(5):
            with dist_autograd.context() as ctx:
                out = pipe(x)
                loss = loss_fn(out, rpc.RRef(target)).to_here()
                dist_autograd.backward(ctx, [loss])
                opt.step(ctx)
                losses.append(float(loss))
        assert losses[-1] < losses[0]
        with pytest.raises(TypeError):
            pipe.cuda()
    rpc.shutdown()


@pytest.mark.parametrize("mode", ["graph", "trace"])
def test_distributed_pipeline_two_workers(mode):
    spawn_ranks(_run, 2, (find_free_port(), mode), backend="gloo", timeout=180.0)
