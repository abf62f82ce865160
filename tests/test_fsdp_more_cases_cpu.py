"""FSDP cases modelled on three reference test files, run as gloo ranks on CPU:

* fairscale tests/nn/data_parallel/test_fsdp_fwd_fwd_bwd_bwd.py: several forwards, then their backwards, all but the last
  inside ``no_sync()`` (what a pipeline schedule does); here the accumulated gradient is also compared with a plain model;
* tests/nn/data_parallel/test_fsdp_input.py: the wrapped module takes a list or a dict;
* tests/nn/data_parallel/test_fsdp_multiple_wrapping.py: a module that already contains FSDP children is wrapped a second
  time after training and gives the same output.
"""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP
from fairscale_b200.nn.data_parallel import TrainingState


class _FFN(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(10, 10), nn.Linear(10, 10)

    def forward(self, x):
        return self.fc2(torch.relu(self.fc1(x)))


def _fwd_fwd_bwd_bwd(rank, world, flatten):
    torch.manual_seed(0)
    plain = _FFN()
    model = FSDP(copy.deepcopy(plain), flatten_parameters=flatten).train()
    torch.manual_seed(10 + rank)
    batches = [torch.rand(10, 10) for _ in range(3)]
    losses = [model(x).sum() for x in batches]
    with model.no_sync():  # only the last backward may reduce
        losses[0].backward()
        losses[1].backward()
    losses[2].backward()
    model.assert_state(TrainingState.IDLE)

    # oracle: the same three losses on the unsharded copy, gradients averaged over the ranks
    for x in batches:
        plain(x).sum().backward()
    want = torch.cat([p.grad.reshape(-1) for p in plain.parameters()])
    dist.all_reduce(want)
    want /= world
    got_local = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
    if flatten:  # one flat shard per rank, padded at the end: gather and cut
        pieces = [torch.zeros_like(got_local) for _ in range(world)]
        dist.all_gather(pieces, got_local)
        got = torch.cat(pieces)[: want.numel()]
        torch.testing.assert_close(got, want)
    else:  # one shard per parameter: compare each against its slice of the full gradient
        offset = 0
        for p_full, p_shard in zip(plain.parameters(), model.parameters()):
            full = want[offset : offset + p_full.numel()]
            offset += p_full.numel()
            pieces = [torch.zeros_like(p_shard.grad.reshape(-1)) for _ in range(world)]
            dist.all_gather(pieces, p_shard.grad.reshape(-1).contiguous())
            torch.testing.assert_close(torch.cat(pieces)[: full.numel()], full)


@pytest.mark.parametrize("flatten", [True, False], ids=["flatten", "no_flatten"])
def test_forwards_then_backwards_with_all_but_the_last_under_no_sync(flatten):
    spawn_ranks(_fwd_fwd_bwd_bwd, 2, (flatten,), backend="gloo")


class _TakesContainer(nn.Module):
    def __init__(self):
        super().__init__()
        self.layer = nn.Linear(4, 4)

    def forward(self, input):
        if isinstance(input, list):
            input = input[0]
        else:
            assert isinstance(input, dict), input
            input = input["in"]
        return self.layer(input)


def _container_input(rank, world, input_cls, config):
    torch.manual_seed(0)
    model = FSDP(_TakesContainer(), **config)
    optim = torch.optim.SGD(model.parameters(), lr=0.1)
    before = model.state_dict()["layer.weight"].clone() if world == 1 else None
    for _ in range(5):
        data = torch.rand(64, 4).requires_grad_(True)
        out = model([data] if input_cls is list else {"in": data})
        out.sum().backward()
        if not config:  # in full precision the gradient reaches the tensor held inside the container; with mixed
            assert data.grad is not None  # precision the root casts its inputs outside autograd, as the reference does
        optim.step()
        optim.zero_grad()
    model.assert_state(TrainingState.IDLE)
    if before is not None:
        assert not torch.equal(before, model.state_dict()["layer.weight"])


@pytest.mark.parametrize("config", [{}, {"mixed_precision": True, "compute_dtype": torch.bfloat16}], ids=["full", "mixed"])
@pytest.mark.parametrize("input_cls", [dict, list])
@pytest.mark.parametrize("world", [1, 2])
def test_input_may_be_a_list_or_a_dict(world, input_cls, config):
    spawn_ranks(_container_input, world, (input_cls, config), backend="gloo")


class _Inner(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layers = nn.Sequential(FSDP(nn.Linear(5, 5), **config))

    def forward(self, x):
        return self.layers(x)


def _wrap_again(rank, world, config):
    torch.manual_seed(0)
    inner = _Inner(config)
    model = FSDP(inner, **config)
    optim = torch.optim.SGD(model.parameters(), lr=0.1)
    for _ in range(3):
        x = torch.rand(1, 5).requires_grad_(True)
        model(x).sum().backward()
        optim.step()
        optim.zero_grad()
    x = torch.rand(1, 5)
    out = model(x)
    model.assert_state(TrainingState.IDLE)
    again = FSDP(inner, **config)  # the inner module keeps its FSDP child
    torch.testing.assert_close(again(x), out)


@pytest.mark.parametrize("world", [1, 2])
@pytest.mark.parametrize("precision", ["full", "mixed"])
@pytest.mark.parametrize("flatten", ["flatten", "no_flatten"])
def test_wrapping_a_trained_module_a_second_time_gives_the_same_output(world, precision, flatten):
    config = {"flatten_parameters": flatten == "flatten"}
    if precision == "mixed":
        config.update(mixed_precision=True, compute_dtype=torch.bfloat16)
    spawn_ranks(_wrap_again, world, (config,), backend="gloo")
