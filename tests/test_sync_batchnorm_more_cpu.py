"""SyncBatchNorm against plain batch norm over the whole batch, for inputs with one, two and three spatial dimensions (cases of
the reference's tests/experimental/nn/test_sync_batchnorm.py on gloo ranks): alone in one process, split over two ranks, under
DistributedDataParallel, in evaluation mode, without affine parameters, with a cumulative average, and called twice inside a
checkpointed block."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.nn.parallel import DistributedDataParallel as DDP

from fairscale_b200.experimental.nn import SyncBatchNorm
from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn import checkpoint_wrapper

SHAPES = {1: (8, 3, 5), 2: (8, 3, 4, 4), 3: (8, 3, 2, 3, 4)}
PLAIN = {1: nn.BatchNorm1d, 2: nn.BatchNorm2d, 3: nn.BatchNorm3d}


def _weights(shape):
    return torch.arange(float(shape[0])).view(-1, *([1] * (len(shape) - 1))) + 1.0


def _parity(rank, world, dims, ddp, affine, momentum):
    torch.manual_seed(0)
    shape = SHAPES[dims]
    per = shape[0] // world
    plain = PLAIN[dims](3, affine=affine, momentum=momentum)
    sync = SyncBatchNorm(3, affine=affine, momentum=momentum)
    if affine:
        with torch.no_grad():
            for m in (plain, sync):
                m.weight.copy_(torch.tensor([0.5, 1.0, 1.5]))
                m.bias.copy_(torch.tensor([0.1, -0.2, 0.3]))
    model = DDP(sync) if ddp and affine else sync
    for step in range(3):
        full = torch.randn(*shape, generator=torch.Generator().manual_seed(step)) * (step + 1) + step
        w = _weights(shape)
        a = full.clone().requires_grad_()
        out_plain = plain(a)
        (out_plain * w).sum().backward()
        b = full[rank * per:(rank + 1) * per].clone().requires_grad_()
        out = model(b)
        (out * w[rank * per:(rank + 1) * per]).sum().backward()
        torch.testing.assert_close(out, out_plain[rank * per:(rank + 1) * per], atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(b.grad, a.grad[rank * per:(rank + 1) * per], atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(sync.running_mean, plain.running_mean, atol=1e-6, rtol=1e-4)
        torch.testing.assert_close(sync.running_var, plain.running_var, atol=1e-6, rtol=1e-4)
        if affine:
            g = sync.weight.grad.clone()
            if not ddp:
                dist.all_reduce(g)          # each rank has the gradient of its rows
            else:
                g = g * world               # DDP averaged them
            torch.testing.assert_close(g, plain.weight.grad, atol=1e-4, rtol=1e-4)
            sync.weight.grad = None
            sync.bias.grad = None
            plain.weight.grad = None
            plain.bias.grad = None
    assert int(sync.num_batches_tracked) == 3
    # evaluation uses the running statistics and needs no communication
    sync.eval()
    plain.eval()
    x = torch.randn(2, *shape[1:], generator=torch.Generator().manual_seed(100 + rank))
    torch.testing.assert_close(sync(x), plain(x), atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("dims", [1, 2, 3])
def test_one_process_equals_batch_norm(dims):
    spawn_ranks(_parity, 1, (dims, False, True, 0.1), backend="gloo")


@pytest.mark.parametrize("dims", [1, 2, 3])
@pytest.mark.parametrize("ddp", [False, True])
def test_two_ranks_equal_batch_norm_over_the_whole_batch(dims, ddp):
    spawn_ranks(_parity, 2, (dims, ddp, True, 0.1), backend="gloo")


@pytest.mark.parametrize("affine,momentum", [(False, 0.1), (True, None), (True, 0.5)])
def test_without_affine_parameters_and_with_other_momenta(affine, momentum):
    spawn_ranks(_parity, 2, (2, False, affine, momentum), backend="gloo")


class _Twice(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(3, 3, 1)
        self.bn = nn.BatchNorm2d(3)

    def forward(self, x):
        return self.bn(self.conv(self.bn(x)))  # the same layer twice


def _checkpointed_twice(rank, world):
    torch.manual_seed(0)
    plain = _Twice()
    sync = SyncBatchNorm.convert_sync_batchnorm(copy.deepcopy(plain))
    assert isinstance(sync.bn, SyncBatchNorm) and sync.bn.weight is not plain.bn.weight
    block = checkpoint_wrapper(sync)
    full = torch.randn(8, 3, 4, 4, generator=torch.Generator().manual_seed(1))
    per = 8 // world
    a = full.clone().requires_grad_()
    plain(a).pow(2).sum().backward()
    b = full[rank * per:(rank + 1) * per].clone().requires_grad_()
    block(b).pow(2).sum().backward()
    torch.testing.assert_close(b.grad, a.grad[rank * per:(rank + 1) * per], atol=1e-4, rtol=1e-3)
    # the replay in backward did not touch the statistics a second time
    assert int(sync.bn.num_batches_tracked) == int(plain.bn.num_batches_tracked) == 2
    torch.testing.assert_close(sync.bn.running_mean, plain.bn.running_mean, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(sync.bn.running_var, plain.bn.running_var, atol=1e-5, rtol=1e-4)


def test_layer_used_twice_inside_a_checkpointed_block():
    spawn_ranks(_checkpointed_twice, 2, (), backend="gloo")


def _conversion(rank, world):
    group = dist.new_group([0, 1])
    net = nn.Sequential(nn.Conv2d(3, 3, 1), nn.BatchNorm2d(3, eps=1e-3, momentum=0.2), nn.Sequential(nn.BatchNorm1d(3, affine=False), nn.ReLU()))
    net[1].running_mean.fill_(0.25)
    out = SyncBatchNorm.convert_sync_batchnorm(net, process_group=group)
    assert out is net and isinstance(net[1], SyncBatchNorm) and isinstance(net[2][0], SyncBatchNorm) and isinstance(net[0], nn.Conv2d)
    assert net[1].eps == 1e-3 and net[1].momentum == 0.2 and float(net[1].running_mean[0]) == 0.25
    assert net[2][0].weight is None and net[2][0].bias is None and net[1].weight is not None
    with pytest.raises(ValueError):
        SyncBatchNorm(3)(torch.zeros(4))  # needs at least (batch, channels)


def test_conversion_keeps_settings_and_statistics():
    spawn_ranks(_conversion, 2, (), backend="gloo")


def _several_calls_per_step(rank, world, nested):
    """The same checkpointed block runs three times in one step (autograd repeats the calls last first), optionally inside an
    outer checkpointed block: every repetition gets the statistics of its own first run."""
    from fairscale_b200.nn.checkpoint import checkpoint_invocations

    torch.manual_seed(0)
    plain = nn.Sequential(nn.Conv2d(3, 3, 1), nn.BatchNorm2d(3))
    sync = SyncBatchNorm.convert_sync_batchnorm(copy.deepcopy(plain))
    block = checkpoint_wrapper(sync)
    if nested:
        outer = checkpoint_wrapper(nn.Sequential(block))
        run = lambda t: outer(t)  # noqa: E731
    else:
        run = block
    per = 4
    g = torch.Generator().manual_seed(1)
    xs = [torch.randn(8, 3, 4, 4, generator=g) * (i + 1) + i for i in range(3)]  # very different statistics per call
    a = [x.clone().requires_grad_() for x in xs]
    sum(plain(t).pow(2).sum() for t in a).backward()
    b = [x[rank * per:(rank + 1) * per].clone().requires_grad_() for x in xs]
    sum(run(t).pow(2).sum() for t in b).backward()
    for got, want in zip(b, a):
        torch.testing.assert_close(got.grad, want.grad[rank * per:(rank + 1) * per], atol=1e-3, rtol=1e-3)
    assert int(sync[1].num_batches_tracked) == int(plain[1].num_batches_tracked) == 3
    torch.testing.assert_close(sync[1].running_var, plain[1].running_var, atol=1e-4, rtol=1e-4)
    assert checkpoint_invocations() == []  # nothing is left running


@pytest.mark.parametrize("nested", [False, True])
def test_block_called_several_times_per_step(nested):
    spawn_ranks(_several_calls_per_step, 2, (nested,), backend="gloo")


def test_every_checkpointed_call_has_its_own_scratch():
    from fairscale_b200.nn.checkpoint import checkpoint_invocations

    seen = []

    class Probe(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(2, 2)

        def forward(self, x):
            stack = checkpoint_invocations()
            scratch = stack[-1]
            scratch.setdefault("visits", []).append(scratch["_mode"])
            seen.append((id(scratch), scratch["_mode"], len(stack)))
            return self.lin(x)

    probe = checkpoint_wrapper(Probe())
    x = torch.randn(3, 2, requires_grad=True)
    (probe(x).sum() + probe(x * 2).sum()).backward()
    first_a, first_b, replay_1, replay_2 = seen
    assert first_a[1] == first_b[1] == "first" and replay_1[1] == replay_2[1] == "replay"
    assert first_a[0] != first_b[0]                      # two calls, two scratch dicts
    assert {replay_1[0], replay_2[0]} == {first_a[0], first_b[0]}  # each repetition finds the dict of its own call
    assert all(depth == 1 for _, _, depth in seen) and checkpoint_invocations() == []
