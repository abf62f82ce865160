"""A small RegNet-like model (residual block with grouped convolution, squeeze-excite branch, batch norms everywhere, a linear
head) under FSDP against DistributedDataParallel on two gloo ranks, over the grid of the reference's
tests/nn/data_parallel/test_fsdp_regnet.py that runs without a GPU: flattened or not, batch norms wrapped on their own by
``auto_wrap_bn`` or not, synchronised batch norm or plain, conversion before or after the wrapping, with and without biases,
in-place ReLU or not.  After three steps the full state dicts - weights, running statistics, step counters - agree."""
import itertools

import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.nn.parallel import DistributedDataParallel as DDP

from fairscale_b200.experimental.nn import SyncBatchNorm
from fairscale_b200.fair_dev.testing.testing import objects_are_equal, spawn_ranks, state_dict_norm
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP
from fairscale_b200.nn.data_parallel import TrainingState, auto_wrap_bn


class _ResBlock(nn.Module):
    def __init__(self, width_in, width_out, inplace):
        super().__init__()
        self.proj = nn.Conv2d(width_in, width_out, (1, 1), (2, 2), bias=False)
        self.bn = nn.BatchNorm2d(width_out)
        self.f = nn.Sequential(
            nn.Sequential(nn.Conv2d(width_in, width_out, (1, 1), (1, 1), bias=False), nn.BatchNorm2d(width_out), nn.ReLU(inplace)),
            nn.Sequential(nn.Conv2d(width_out, width_out, (3, 3), (2, 2), (1, 1), groups=2, bias=False), nn.BatchNorm2d(width_out), nn.ReLU(inplace)),
            _SqueezeExcite(width_out, inplace),
            nn.Conv2d(width_out, width_out, (1, 1), (1, 1), bias=False),
            nn.BatchNorm2d(width_out),
        )
        self.relu = nn.ReLU()

    def forward(self, x):
        return self.relu(self.bn(self.proj(x)) + self.f(x))


class _SqueezeExcite(nn.Module):
    def __init__(self, width, inplace):
        super().__init__()
        self.pool = nn.AdaptiveAvgPool2d((1, 1))
        self.gate = nn.Sequential(nn.Conv2d(width, 2, (1, 1), bias=False), nn.ReLU(inplace), nn.Conv2d(2, width, (1, 1), bias=False), nn.Sigmoid())

    def forward(self, x):
        return x * self.gate(self.pool(x))


class _Model(nn.Module):
    def __init__(self, conv_bias, linear_bias, inplace):
        super().__init__()
        torch.manual_seed(0)
        self.trunk = nn.Sequential()
        self.trunk.add_module("stem", nn.Sequential(nn.Conv2d(2, 4, (3, 3), (2, 2), (1, 1), bias=conv_bias), nn.BatchNorm2d(4), nn.ReLU(inplace)))
        self.trunk.add_module("any_stage_block1", nn.Sequential(_ResBlock(4, 8, inplace)))
        self.head = nn.Sequential(
            nn.Sequential(nn.Linear(32, 16, bias=linear_bias), nn.ReLU(), nn.Linear(16, 8, bias=linear_bias)), nn.Linear(8, 15, bias=False)
        )

    def forward(self, x):
        return self.head(self.trunk(x).flatten(1))


# the settings auto_wrap_bn uses by default, plus the CPU as compute device
_BN_CONFIG = dict(mixed_precision=False, flatten_parameters=False, reshard_after_forward=False, bucket_cap_mb=0, force_input_to_fp32=False,
                  compute_device=torch.device("cpu"))


def _train(model, rank, iterations=3):
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(100 + rank)
    for _ in range(iterations):
        x = torch.rand(4, 2, 8, 8, generator=g)
        loss = nn.functional.cross_entropy(model(x), torch.zeros(4, dtype=torch.long))
        loss.backward()
        opt.step()
        opt.zero_grad()


def _worker(rank, world, flatten, wrap_bn, sync_bn, convert_first, conv_bias, linear_bias, inplace):
    make = lambda: _Model(conv_bias, linear_bias, inplace)  # noqa: E731
    before = state_dict_norm(make().state_dict())

    ref = make()
    if sync_bn:
        ref = SyncBatchNorm.convert_sync_batchnorm(ref)
    ref = DDP(ref, broadcast_buffers=True)
    _train(ref, rank)
    want = ref.module.state_dict()
    assert state_dict_norm(want) != before  # it did train

    model = make()
    steps = [lambda m: SyncBatchNorm.convert_sync_batchnorm(m) if sync_bn else m,
             lambda m: auto_wrap_bn(m, single_rank_pg=False, fsdp_config=_BN_CONFIG) if wrap_bn else m]
    for step in (steps if convert_first else reversed(steps)):
        model = step(model)
    model = FSDP(model, flatten_parameters=flatten, compute_device=torch.device("cpu"))
    if wrap_bn:
        assert sum(isinstance(m, FSDP) for m in model.modules()) == 1 + 5  # the root and one wrapper per batch norm
    _train(model, rank)
    model.assert_state(TrainingState.IDLE)
    got = model.state_dict()
    assert set(got) == set(want)
    if sync_bn or rank == 0:  # without synchronisation every rank has its own running statistics; DDP broadcasts rank 0's
        for k in want:
            if "running_" in k and not sync_bn and rank != 0:
                continue
            torch.testing.assert_close(got[k], want[k], atol=1e-5, rtol=1e-4, msg=lambda m, k=k: f"{k}: {m}")
    dist.barrier()


_GRID = [
    # flatten, wrap_bn, sync_bn, convert_first, conv_bias, linear_bias, inplace
    (True, False, False, True, True, True, False),
    (True, True, False, True, False, True, True),
    (False, True, False, True, True, False, False),
    (False, False, False, True, False, False, True),
    (True, True, True, True, True, True, True),
    (True, True, True, False, False, True, False),
    (False, True, True, False, True, False, True),
    (True, False, True, True, True, True, False),
    (False, False, True, True, False, False, False),
]


@pytest.mark.parametrize("flatten,wrap_bn,sync_bn,convert_first,conv_bias,linear_bias,inplace", _GRID)
def test_regnet_like_model_matches_ddp(flatten, wrap_bn, sync_bn, convert_first, conv_bias, linear_bias, inplace):
    spawn_ranks(_worker, 2, (flatten, wrap_bn, sync_bn, convert_first, conv_bias, linear_bias, inplace), backend="gloo")


def test_the_grid_touches_every_value_of_every_axis():
    assert all({row[i] for row in _GRID} == {True, False} for i in range(7))
    assert len(set(_GRID)) == len(_GRID) and len(list(itertools.product([True, False], repeat=7))) == 128
