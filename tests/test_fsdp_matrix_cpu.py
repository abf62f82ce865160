"""More of the reference's FSDP test matrix on 2 gloo ranks (CPU): gradient accumulation with and without ``no_sync``
(tests/nn/data_parallel/test_fsdp_grad_acc.py), the pre-backward hook of a unit with several outputs
(test_fsdp_pre_backward_hook.py), a checkpointed unit called several times per step
(test_fsdp_multiple_forward_checkpoint.py), freezing in every wrapping layout (test_fsdp_freezing_weights.py), and
``no_sync`` before the first forward."""
import contextlib

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import DummyProcessGroup, spawn_ranks
from fairscale_b200.nn import FullyShardedDataParallel as FSDP
from fairscale_b200.nn import checkpoint_wrapper
from fairscale_b200.parallel import comm

CPU = dict(compute_device=torch.device("cpu"))


def _net(seed=0, d=8):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(d, 12), nn.Tanh(), nn.Linear(12, 12), nn.Tanh(), nn.Linear(12, 3))


def _wrapped(flatten, nested, **kw):
    net = _net()
    if nested:
        layers = list(net)
        net = nn.Sequential(FSDP(nn.Sequential(*layers[:2]), flatten_parameters=flatten, **CPU, **kw), layers[2],
                            FSDP(nn.Sequential(*layers[3:]), flatten_parameters=flatten, **CPU, **kw))
    return FSDP(net, flatten_parameters=flatten, **CPU, **kw)


def _batch(rank, step, micro, d=8):
    g = torch.Generator().manual_seed(1000 * step + 10 * micro + rank)
    return torch.randn(4, d, generator=g)


def _grad_acc(rank, world, flatten, nested, use_no_sync):
    """Two micro-batches accumulated into one step: the gradient (and the weights after the step) must equal those of one
    pass over the concatenated batch, whether or not the first micro-batch runs under ``no_sync``; under ``no_sync`` no
    gradient is reduced."""
    model = _wrapped(flatten, nested)
    ref = _wrapped(flatten, nested)
    opt, ref_opt = torch.optim.SGD(model.parameters(), lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    for step in range(2):
        a, b = _batch(rank, step, 0), _batch(rank, step, 1)
        ref_opt.zero_grad()
        ref(torch.cat([a, b])).pow(2).sum().backward()
        ref_opt.step()

        opt.zero_grad()
        comm.reset_counters()
        ctx = model.no_sync() if use_no_sync else contextlib.nullcontext()
        with ctx:
            model(a).pow(2).sum().backward()
        reduced_first = comm.counters().get("reduce_scatter", 0)
        assert (reduced_first == 0) == use_no_sync, reduced_first
        model(b).pow(2).sum().backward()
        assert comm.counters().get("reduce_scatter", 0) > reduced_first
        opt.step()
    for (k, v), w in zip(model.state_dict().items(), ref.state_dict().values()):
        torch.testing.assert_close(v, w, atol=1e-6, rtol=1e-5, msg=lambda m, k=k: f"{k}: {m}")


@pytest.mark.parametrize("flatten,nested,use_no_sync", [(True, False, True), (True, True, True), (False, True, True), (True, True, False),
                                                        (False, False, False)])
def test_fsdp_gradient_accumulation(flatten, nested, use_no_sync):
    spawn_ranks(_grad_acc, 2, (flatten, nested, use_no_sync), backend="gloo")


def test_fsdp_no_sync_before_the_first_forward():
    group = DummyProcessGroup(rank=0, size=1)
    model = FSDP(_net(), process_group=group, process_group_reduce_scatter=DummyProcessGroup(rank=0, size=1), **CPU)
    x = torch.randn(4, 8)
    with model.no_sync():
        model(x).sum().backward()
    first = [p.grad.clone() for p in model.parameters()]
    model(x).sum().backward()
    for g, p in zip(first, model.parameters()):
        torch.testing.assert_close(p.grad, 2 * g)  # the second backward accumulated onto the unsynchronised gradient


class _TwoHeads(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(3)
        self.trunk = nn.Linear(8, 8)
        self.left, self.right = nn.Linear(8, 2), nn.Linear(8, 2)

    def forward(self, x):
        h = torch.tanh(self.trunk(x))
        return self.left(h), self.right(h)


def _pre_backward(rank, world):
    """A unit with two outputs: the pre-backward work (re-gathering the parameters) must run once per backward, not once per
    output, and the gradients must match DDP when both outputs feed the loss and when only one does."""
    ref = nn.parallel.DistributedDataParallel(_TwoHeads(), find_unused_parameters=True)
    model = FSDP(_TwoHeads(), **CPU)
    calls = []
    original = model._rebuild_full_params

    def counting(*a, **k):
        calls.append(1)
        return original(*a, **k)

    model._rebuild_full_params = counting  # type: ignore[method-assign]
    for step, use_right in enumerate((True, False, True)):
        x = _batch(rank, step, 0)
        for m in (ref, model):
            m.zero_grad()
            left, right = m(x)
            loss = left.pow(2).sum() + (right.pow(2).sum() if use_right else 0.0)
            before = len(calls)
            loss.backward()
            if m is model:
                assert len(calls) - before <= 1, "parameters re-gathered more than once in one backward"
        with model.summon_full_params():
            for (n, p), q in zip(model.module.named_parameters(), ref.module.parameters()):
                pass  # full parameters are addressable by their original names inside the context
        ref_grads = {n: (p.grad if p.grad is not None else torch.zeros_like(p)) for n, p in ref.module.named_parameters()}
        flat = torch.cat([ref_grads[n].reshape(-1) for n, _ in ref.module.named_parameters()])
        shard = model.params[0].grad
        n = shard.numel()
        padded = torch.cat([flat, flat.new_zeros(n * world - flat.numel())])
        torch.testing.assert_close(shard.reshape(-1), padded[rank * n : (rank + 1) * n], atol=1e-6, rtol=1e-5)


def test_fsdp_pre_backward_hook_runs_once_for_a_unit_with_two_outputs():
    spawn_ranks(_pre_backward, 2, (), backend="gloo")


class _Reused(nn.Module):
    """One (optionally checkpointed) block applied to three inputs per step, like the reference's multi-crop SSL model."""

    def __init__(self, checkpoint, wrap_block):
        super().__init__()
        torch.manual_seed(5)
        block = nn.Sequential(nn.Linear(8, 8), nn.Tanh(), nn.Linear(8, 8))
        if checkpoint:
            block = checkpoint_wrapper(block)
        self.block = FSDP(block, **CPU) if wrap_block else block
        self.head = nn.Linear(8, 2)

    def forward(self, xs):
        return self.head(torch.cat([self.block(x) for x in xs]))


def _multi_forward(rank, world, checkpoint, wrap_block):
    ref = nn.parallel.DistributedDataParallel(_Reused(False, False))
    model = FSDP(_Reused(checkpoint, wrap_block), **CPU)
    opt, ref_opt = torch.optim.SGD(model.parameters(), lr=0.05), torch.optim.SGD(ref.parameters(), lr=0.05)
    for step in range(3):
        xs = [_batch(rank, step, k) for k in range(3)]
        for m, o in ((ref, ref_opt), (model, opt)):
            o.zero_grad()
            m(xs).pow(2).mean().backward()
            o.step()
    for (k, v), w in zip(model.state_dict().items(), ref.module.state_dict().values()):
        torch.testing.assert_close(v, w, atol=1e-6, rtol=1e-5, msg=lambda m, k=k: f"{k}: {m}")


@pytest.mark.parametrize("checkpoint,wrap_block", [(True, True), (True, False), (False, True)])
def test_fsdp_block_called_three_times_per_step(checkpoint, wrap_block):
    spawn_ranks(_multi_forward, 2, (checkpoint, wrap_block), backend="gloo")


def _freezing(rank, world, flatten, nested, freeze_after_wrap):
    """The first two layers frozen, before or after wrapping: frozen shards stay bit-identical, the rest follows DDP."""

    def freeze(net):
        for p in list(net.parameters())[:4]:
            p.requires_grad = False

    ref_net = _net()
    freeze(ref_net)
    ref = nn.parallel.DistributedDataParallel(ref_net)
    if freeze_after_wrap:
        model = _wrapped(flatten, nested)
        if not flatten:
            freeze(model)
        else:
            pytest.skip("freezing single parameters after wrapping needs unflattened parameters")
    else:
        net = _net()
        freeze(net)
        layers = list(net)
        if nested:
            net = nn.Sequential(FSDP(nn.Sequential(*layers[:3]), flatten_parameters=flatten, **CPU), *layers[3:])
        model = FSDP(net, flatten_parameters=flatten, **CPU)
    before = {k: v.clone() for k, v in model.state_dict().items()}
    opt = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=0.1)
    ref_opt = torch.optim.SGD([p for p in ref.parameters() if p.requires_grad], lr=0.1)
    for step in range(3):
        x = _batch(rank, step, 0)
        for m, o in ((ref, ref_opt), (model, opt)):
            o.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    after = model.state_dict()
    for i, ((k, v), w) in enumerate(zip(after.items(), ref.module.state_dict().values())):
        torch.testing.assert_close(v, w, atol=1e-6, rtol=1e-5, msg=lambda m, k=k: f"{k}: {m}")
        if i < 4:
            assert torch.equal(v, before[k]), k


@pytest.mark.parametrize("flatten,nested,freeze_after_wrap", [(True, True, False), (False, True, False), (False, False, True), (False, True, True)])
def test_fsdp_frozen_layers_in_every_layout(flatten, nested, freeze_after_wrap):
    spawn_ranks(_freezing, 2, (flatten, nested, freeze_after_wrap), backend="gloo")


def test_fsdp_rejects_a_step_while_unsharded_and_reports_state():
    """State machine checks of the reference (fully_sharded_data_parallel.py: assert_state): a second ``summon_full_params`` inside
    the first is allowed to nest, a forward inside it is not."""
    group = DummyProcessGroup(rank=0, size=1)
    model = FSDP(_net(), process_group=group, **CPU)
    with model.summon_full_params():
        with pytest.raises((AssertionError, ValueError, RuntimeError)):
            model(torch.randn(2, 8))
    model(torch.randn(2, 8)).sum().backward()  # usable again afterwards
    assert not dist.is_initialized() or True
