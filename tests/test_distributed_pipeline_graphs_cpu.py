"""RPC pipeline over module graphs that are not a chain, on CPU workers (cases of the reference's
tests/experimental/nn/test_multiprocess_pipe.py): one worker (construction, forward, chunked forward), two workers with every
checkpoint mode, a layer with two outputs feeding two branches on different workers that meet again in a layer with two
inputs - built by hand and extracted from a traced model - and training through distributed autograd."""
import os

import pytest
import torch
from torch import nn

from fairscale_b200.fair_dev.testing.testing import find_free_port, spawn_ranks


class ConcatenateTensors(nn.Module):
    def forward(self, *inputs):
        return torch.cat(inputs, dim=1)


class SplitTensors(nn.Module):
    def forward(self, input):
        return torch.split(input, (input.shape[1] + 1) // 2, dim=1)


class ShardedLinearLayer(nn.Module):
    """split -> one small linear layer per shard (on different workers) -> concatenate"""

    def __init__(self, input_device, shard_devices, output_device):
        from torch.distributed.nn import RemoteModule

        super().__init__()
        self.split = RemoteModule(input_device, SplitTensors, (), {})
        self.linear_layers_2 = nn.ModuleList([RemoteModule(d, nn.Linear, (2, 2), {}) for d in shard_devices])
        self.concatenate = RemoteModule(output_device, ConcatenateTensors, ())

    def forward(self, input):
        shards = self.split(input)
        return self.concatenate(*[layer(shards[i]) for i, layer in enumerate(self.linear_layers_2)])


def _partitions(graph, pipe):
    return [[graph.nodes.index(n) for n in p.nodes] for p in pipe.partitions]


def _train_two_steps(pipe, x, n_params):
    import torch.distributed.autograd as dist_autograd
    from torch.distributed import rpc
    from torch.distributed.optim import DistributedOptimizer

    from fairscale_b200.experimental.nn.distributed_pipeline import DistributedLoss

    rrefs = pipe.parameter_rrefs()
    assert len(rrefs) == n_params
    opt = DistributedOptimizer(torch.optim.SGD, rrefs, lr=0.05)
    criterion = DistributedLoss(nn.MSELoss)
    losses = []
    for _ in range(2):
        with dist_autograd.context() as ctx:
            loss = criterion(pipe(x), rpc.RRef(x))
            losses.append(loss)
            loss.backward(ctx)
            opt.step(ctx)
    first, second = (float(l.to_here()) for l in losses)
    assert first > second, (first, second)


def _case_single_worker(devices):
    from torch.distributed.nn import RemoteModule

    from fairscale_b200.experimental.nn.distributed_pipeline import DistributedPipeline, PipelineModulesGraph

    def chain(n_layers, chunks):
        graph = PipelineModulesGraph()
        graph.add_sequence([RemoteModule(devices[0], nn.Linear, (4, 4), {}) for _ in range(n_layers)], [0])
        return DistributedPipeline(graph, chunks=chunks)

    pipe = chain(1, 1)
    assert len(pipe.partitions) == 1
    assert len(chain(3, 1).partitions) == 1  # consecutive layers on one device share a partition
    torch.manual_seed(3)
    x = torch.randn(8, 4)
    weight, bias = [r.to_here() for r in pipe.parameter_rrefs()]
    torch.testing.assert_close(pipe(x).to_here(), x @ weight.t() + bias)
    # chunked: rows are processed in pieces and put together again in order
    chunked = chain(1, 4)
    weight, bias = [r.to_here() for r in chunked.parameter_rrefs()]
    out = chunked(x).to_here()
    assert out.shape == (8, 4)
    torch.testing.assert_close(out, x @ weight.t() + bias)
    # fewer rows than chunks
    assert chunked(x[:2]).to_here().shape == (2, 4)


def _case_checkpoint_modes(devices):
    from torch.distributed.nn import RemoteModule

    from fairscale_b200.experimental.nn.distributed_pipeline import DistributedPipeline, PipelineModulesGraph

    torch.manual_seed(3)
    x = torch.randn(8, 4)
    for mode in ("never", "always", "except_last"):
        layers = [RemoteModule(devices[0], nn.Linear, (4, 4), {}), RemoteModule(devices[0], nn.ReLU, (), {}),
                  RemoteModule(devices[1], nn.Linear, (4, 4), {}), RemoteModule(devices[1], nn.ReLU, (), {})]
        graph = PipelineModulesGraph()
        graph.add_sequence(layers, [0])
        pipe = DistributedPipeline(graph, chunks=4, checkpoint=mode)
        assert _partitions(graph, pipe) == [[0, 1], [2, 3]]
        w1, b1, w2, b2 = [r.to_here() for r in pipe.parameter_rrefs()]
        want = torch.relu(torch.relu(x @ w1.t() + b1) @ w2.t() + b2)
        torch.testing.assert_close(pipe(x).to_here(), want)
        _train_two_steps(pipe, x, 4)
    with pytest.raises(ValueError):
        DistributedPipeline(graph, chunks=0)
    with pytest.raises(ValueError):
        DistributedPipeline(graph, chunks=2, checkpoint="sometimes")


def _case_branches_by_hand(devices):
    from torch.distributed.nn import RemoteModule

    from fairscale_b200.experimental.nn.distributed_pipeline import DistributedPipeline, PipelineModulesGraph

    torch.manual_seed(3)
    x = torch.randn(8, 4)
    first = RemoteModule(devices[0], nn.Linear, (4, 4), {})
    split = RemoteModule(devices[0], SplitTensors, (), {})
    branches = [RemoteModule(devices[0], nn.Linear, (2, 2), {}), RemoteModule(devices[1], nn.Linear, (2, 2), {})]
    concat = RemoteModule(devices[1], ConcatenateTensors, ())
    graph = PipelineModulesGraph()
    graph.add_sequence([first, split], [0], 2)           # the last layer of the sequence has two outputs
    for i, layer in enumerate(branches):
        graph.add_layer(layer, [(split, i)])             # each branch reads one of them
    graph.add_layer(concat, branches)
    pipe = DistributedPipeline(graph, chunks=4)
    assert _partitions(graph, pipe) == [[0, 1], [2], [3], [4]]
    w, b, wa, ba, wb, bb = [r.to_here() for r in pipe.parameter_rrefs()]
    h = x @ w.t() + b
    want = torch.cat([h[:, :2] @ wa.t() + ba, h[:, 2:] @ wb.t() + bb], dim=1)
    torch.testing.assert_close(pipe(x).to_here(), want)
    _train_two_steps(pipe, x, 6)


def _case_branches_traced(devices):
    from torch.distributed.nn import RemoteModule

    from fairscale_b200.experimental.nn.distributed_pipeline import DistributedPipeline, make_graph

    torch.manual_seed(3)
    x = torch.randn(8, 4)
    model = nn.Sequential(RemoteModule(devices[0], nn.Linear, (4, 4), {}), ShardedLinearLayer(devices[0], devices, devices[1]),
                          RemoteModule(devices[0], nn.Linear, (4, 4), {}))
    graph = make_graph(model)
    pipe = DistributedPipeline(graph, chunks=4)
    assert _partitions(graph, pipe) == [[0, 1], [2], [3], [4], [5]]
    assert pipe(x).to_here().shape == (8, 4)
    _train_two_steps(pipe, x, 8)


_CASES = {"single_worker": (_case_single_worker, 1), "checkpoint_modes": (_case_checkpoint_modes, 2),
          "branches_by_hand": (_case_branches_by_hand, 2), "branches_traced": (_case_branches_traced, 2)}


def _worker(rank, world, port, case):
    from torch.distributed import rpc

    # every worker imports the package before it serves requests: the request threads of an RPC agent would otherwise import it
    # concurrently while unpickling their first calls
    import fairscale_b200.experimental.nn.distributed_pipeline  # noqa: F401

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    rpc.init_rpc(f"worker{rank}", rank=rank, world_size=world,
                 rpc_backend_options=rpc.TensorPipeRpcBackendOptions(init_method=f"tcp://127.0.0.1:{port}", _transports=["uv"]))
    if rank == 0:
        _CASES[case][0]([f"worker{r}/cpu" for r in range(world)])
    rpc.shutdown()


@pytest.mark.parametrize("case", list(_CASES))
def test_distributed_pipeline_case(case):
    spawn_ranks(_worker, _CASES[case][1], (find_free_port(), case), backend="gloo", timeout=240.0)
