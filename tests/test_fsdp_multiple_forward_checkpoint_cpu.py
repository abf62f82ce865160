"""FSDP units that run three times per step on inputs of different sizes, with and without checkpoint_wrapper around them
(cases of the reference's tests/nn/data_parallel/test_fsdp_multiple_forward_checkpoint.py on gloo ranks, full precision):
every combination gives the losses of DistributedDataParallel, step by step - for two model shapes, plain and synchronised
batch norm, flattened or not, batch norms in wrappers of their own or not, gradients bucketed or not, and with the
gradient division moved entirely after the reduction."""
import contextlib

import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.nn.parallel import DistributedDataParallel as DDP

from fairscale_b200.experimental.nn import SyncBatchNorm
from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn import checkpoint_wrapper
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP
from fairscale_b200.nn.data_parallel import auto_wrap_bn
from fairscale_b200.nn.wrap import enable_wrap, wrap

CPU = torch.device("cpu")


class _Model(nn.Module):
    def __init__(self, deep):
        super().__init__()
        torch.manual_seed(0)
        self.block1 = nn.Sequential(nn.Conv2d(3, 4, kernel_size=3), nn.BatchNorm2d(4), nn.ReLU(inplace=True))
        if deep:
            self.block2 = nn.Sequential(nn.Conv2d(4, 4, kernel_size=3), nn.BatchNorm2d(4), nn.ReLU(inplace=False))
            self.block3 = nn.Sequential(nn.Conv2d(4, 8, kernel_size=3), nn.BatchNorm2d(8), nn.ReLU(inplace=True))
            self.head = nn.Sequential(nn.AdaptiveAvgPool2d(output_size=(1, 1)), nn.Flatten(), nn.Linear(8, 10))
            self.blocks = ["block1", "block2", "block3"]
        else:
            self.block2 = nn.Sequential(nn.Conv2d(4, 8, kernel_size=3), nn.BatchNorm2d(8), nn.ReLU(inplace=True),
                                        nn.AdaptiveAvgPool2d(output_size=(1, 1)), nn.Flatten())
            self.head = nn.Linear(8, 10)
            self.blocks = ["block1", "block2"]

    def _one(self, x):
        for name in self.blocks:
            x = getattr(self, name)(x)
        return self.head(x)

    def forward(self, x):
        return self._one(x) if isinstance(x, torch.Tensor) else torch.cat([self._one(e) for e in x], dim=0)


def _build(deep, sync_bn, with_fsdp, with_checkpoint, flatten, wrap_bn, bucket_cap_mb):
    model = _Model(deep)
    bn_config = None
    if sync_bn:
        model = SyncBatchNorm.convert_sync_batchnorm(model)
        bn_config = dict(mixed_precision=False, flatten_parameters=False, reshard_after_forward=False, bucket_cap_mb=0, force_input_to_fp32=True,
                         compute_device=CPU)
    elif wrap_bn:
        bn_config = dict(mixed_precision=False, flatten_parameters=False, reshard_after_forward=False, bucket_cap_mb=0, force_input_to_fp32=False,
                         compute_device=CPU)
    if with_fsdp and wrap_bn:
        for name in model.blocks:
            setattr(model, name, auto_wrap_bn(getattr(model, name), single_rank_pg=False, fsdp_config=bn_config))
    if with_checkpoint:
        for name in model.blocks[1:]:
            setattr(model, name, checkpoint_wrapper(getattr(model, name)))
    if with_fsdp:
        with enable_wrap(wrapper_cls=FSDP, flatten_parameters=flatten, bucket_cap_mb=bucket_cap_mb, compute_device=CPU):
            for name in model.blocks + ["head"]:
                setattr(model, name, wrap(getattr(model, name)))
        model = FSDP(model, flatten_parameters=flatten, bucket_cap_mb=bucket_cap_mb, compute_device=CPU)
        model.set_gradient_divide_factors(1.0, 2.0, True)  # nothing before the reduction, the world size after it
    return model


def _losses(rank, world, model, is_ddp):
    g = torch.Generator().manual_seed(7)
    batch = [torch.randn(2, 3, 16, 16, generator=g), torch.randn(2, 3, 9, 9, generator=g), torch.randn(2, 3, 9, 9, generator=g)]
    batch = [b + rank for b in batch]  # ranks see different data
    target = torch.tensor([0, 1, 2, 3, 4, 5])
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    out = []
    with (model.no_sync() if is_ddp else contextlib.nullcontext()):
        for _ in range(3):
            loss = nn.functional.cross_entropy(model(batch), target)
            out.append(float(loss))
            opt.zero_grad()
            loss.backward()
            if is_ddp:  # the reduction by hand, so that both arms divide after summing
                for p in model.parameters():
                    dist.all_reduce(p.grad)
                    p.grad.div_(world)
            opt.step()
    return out


def _worker(rank, world, deep, sync_bn, flatten, wrap_bn):
    want = _losses(rank, world, DDP(_build(deep, sync_bn, False, False, flatten, wrap_bn, 0)), True)
    assert want[-1] != want[0]
    for with_checkpoint in (False, True):
        for bucket_cap_mb in (0, 25):
            model = _build(deep, sync_bn, True, with_checkpoint, flatten, wrap_bn, bucket_cap_mb)
            got = _losses(rank, world, model, False)
            for step, (a, b) in enumerate(zip(got, want)):
                assert abs(a - b) <= 1e-5 * max(1.0, abs(b)), (with_checkpoint, bucket_cap_mb, step, got, want)
    dist.barrier()


_LAYOUTS = [(True, True, False), (True, False, False), (False, True, False), (False, False, False), (True, True, True), (False, True, True)]


@pytest.mark.parametrize("deep", [False, True], ids=["two_blocks", "three_blocks"])
@pytest.mark.parametrize("flatten,wrap_bn,sync_bn", _LAYOUTS)
def test_units_run_three_times_per_step_with_and_without_checkpointing(deep, flatten, wrap_bn, sync_bn):
    spawn_ranks(_worker, 2, (deep, sync_bn, flatten, wrap_bn), backend="gloo")
