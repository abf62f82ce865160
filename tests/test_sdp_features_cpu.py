"""ShardedDataParallel behaviours around the training loop, on gloo CPU ranks (the cases of the reference's
tests/nn/data_parallel/test_sharded_ddp_features.py): container inputs, the DistributedDataParallel-like attributes,
attribute forwarding to the wrapped module, refusing gradients that require gradients, parameters of mixed dtypes,
train / eval switches, trainability changes with and without automatic refresh, several process groups, a module moved
with ``.to()``, and a grid of step configurations against DistributedDataParallel."""
import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.data_parallel import ShardedDataParallel
from fairscale_b200.optim import OSS


def _mlp(seed=0, d=6, with_buffer=False):
    torch.manual_seed(seed)
    net = nn.Sequential(nn.Linear(d, 9), nn.Tanh(), nn.Linear(9, 9), nn.Tanh(), nn.Linear(9, 2))
    if with_buffer:
        net.register_buffer("calls", torch.zeros(1))
    return net


def _data(rank, step, d=6):
    g = torch.Generator().manual_seed(97 * step + rank)
    return torch.randn(5, d, generator=g)


def _sdp(model, buffer_size=0, momentum=0.9, **kw):
    oss = OSS(model.parameters(), optim=torch.optim.SGD, lr=0.05, momentum=momentum)
    return ShardedDataParallel(model, oss, reduce_buffer_size=buffer_size, **kw), oss


class _TwoInputs(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(2)
        self.a, self.b = nn.Linear(6, 4), nn.Linear(6, 4)

    def forward(self, pair, extra=None):
        x, y = pair
        out = self.a(x) + self.b(y)
        return out if extra is None else out + extra["bias"]


def _containers(rank, world, buffer_size):
    model, oss = _sdp(_TwoInputs(), buffer_size)
    x, y = _data(rank, 0), _data(rank, 1)
    out = model((x, y), extra={"bias": torch.ones(4)})
    out.sum().backward()
    oss.step()
    assert out.shape == (5, 4)


@pytest.mark.parametrize("buffer_size", [0, 2**16])
def test_sdp_accepts_tuples_and_keyword_containers(buffer_size):
    spawn_ranks(_containers, 2, (buffer_size,), backend="gloo")


def _attributes(rank, world):
    net = _mlp()
    net.banana = "sweet"
    model, _ = _sdp(net)
    # what DistributedDataParallel users look at
    assert model.is_multi_device_module is False and model.device_type == "cpu" and model.module is net
    # unknown attributes fall through to the wrapped module, and only to it
    assert model.banana == "sweet" and not hasattr(model, "orange")

    # a gradient that itself requires grad cannot be reduced in place: refuse at the first forward
    net = _mlp()
    first = next(net.parameters())
    first.grad = torch.zeros_like(first).requires_grad_()
    model, _ = _sdp(net)
    with pytest.raises(RuntimeError):
        model(_data(rank, 0))


def test_sdp_attributes_forwarding_and_grad_of_grad_refusal():
    spawn_ranks(_attributes, 1, (), backend="gloo")


def _mixed_dtypes(rank, world, buffer_size):
    # parameters of two dtypes: buckets take the dtype of their first member, the rest is reduced parameter by parameter
    net = _mlp()
    net[2] = net[2].double()
    net.insert(2, _Cast(torch.float64))
    net.insert(4, _Cast(torch.float32))
    ref = nn.parallel.DistributedDataParallel(_same_as(net))
    model, oss = _sdp(net, buffer_size)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    for step in range(3):
        x = _data(rank, step)
        for m, o in ((ref, ref_opt), (model, oss)):
            m.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    for a, b in zip(ref.module.parameters(), net.parameters()):
        torch.testing.assert_close(b, a, atol=1e-6, rtol=1e-5)


class _Cast(nn.Module):
    def __init__(self, dtype):
        super().__init__()
        self.dtype = dtype

    def forward(self, x):
        return x.to(self.dtype)


def _same_as(net):
    import copy

    return copy.deepcopy(net)


@pytest.mark.parametrize("buffer_size", [0, 2**16])
def test_sdp_parameters_of_two_dtypes(buffer_size):
    spawn_ranks(_mixed_dtypes, 2, (buffer_size,), backend="gloo")


def _train_eval(rank, world):
    model, _ = _sdp(_mlp())
    x = _data(rank, 0)
    model(x).sum().backward()
    model.zero_grad()
    model.eval()
    model(x)  # no backward follows: nothing may be left waiting for a reduction
    assert all(p.grad is None or float(p.grad.norm()) < 1e-6 for p in model.parameters())
    model.train()
    model(x).sum().backward()
    # gradients live on the rank that owns the parameter's optimizer state only
    owned = [p for p in model.parameters() if p.grad is not None]
    assert owned and all(float(p.grad.norm()) > 0.0 for p in owned)


def test_sdp_train_eval_train():
    spawn_ranks(_train_eval, 2, (), backend="gloo")


def _trainability(rank, world, auto_refresh, buffer_size):
    """Freeze the first layer after two steps: with automatic refresh the wrapper notices at the next forward, without it
    ``refresh_trainable()`` has to be called; afterwards the frozen weights stay put and the rest follows DDP."""
    ref_net, net = _mlp(), _mlp()
    ref = nn.parallel.DistributedDataParallel(ref_net, find_unused_parameters=True)
    # no momentum: the wrapper's zero_grad keeps zero-filled gradients (they are views of its buckets), and a momentum
    # buffer would go on moving a frozen parameter whose gradient is zero rather than absent
    model, oss = _sdp(net, buffer_size, momentum=0.0, auto_refresh_trainable=auto_refresh)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    frozen_at = None
    for step in range(5):
        if step == 2:
            for m in (ref_net, net):
                for p in m[0].parameters():
                    p.requires_grad = False
            if not auto_refresh:
                model.refresh_trainable()
            frozen_at = [p.detach().clone() for p in net[0].parameters()]
        x = _data(rank, step)
        for m, o in ((ref, ref_opt), (model, oss)):
            m.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    for a, b in zip(frozen_at, net[0].parameters()):
        assert torch.equal(a, b)
    for a, b in zip(ref_net.parameters(), net.parameters()):
        torch.testing.assert_close(b, a, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("auto_refresh,buffer_size", [(True, 0), (True, 2**16), (False, 2**16)])
def test_sdp_freezing_in_the_middle_of_training(auto_refresh, buffer_size):
    spawn_ranks(_trainability, 2, (auto_refresh, buffer_size), backend="gloo")


def _groups(rank, world, buffer_size):
    """Ranks {0, 1} and {2, 3} train independent replicas in their own process groups."""
    groups = [dist.new_group(ranks=[0, 1]), dist.new_group(ranks=[2, 3])]
    mine = groups[rank // 2]
    net = _mlp(seed=rank // 2)
    oss = OSS(net.parameters(), optim=torch.optim.SGD, group=mine, lr=0.05)
    model = ShardedDataParallel(net, oss, process_group=mine, reduce_buffer_size=buffer_size)
    ref_net = _mlp(seed=rank // 2)
    ref = nn.parallel.DistributedDataParallel(ref_net, process_group=mine)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    for step in range(3):
        x = _data(rank, step)
        for m, o in ((ref, ref_opt), (model, oss)):
            m.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    for a, b in zip(ref_net.parameters(), net.parameters()):
        torch.testing.assert_close(b, a, atol=1e-6, rtol=1e-5)
    # the two replicas really were independent
    flat = torch.cat([p.detach().reshape(-1) for p in net.parameters()])
    everyone = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(everyone, flat)
    assert torch.equal(everyone[0], everyone[1]) and torch.equal(everyone[2], everyone[3]) and not torch.equal(everyone[0], everyone[2])


@pytest.mark.parametrize("buffer_size", [0, 2**16])
def test_sdp_in_two_process_groups(buffer_size):
    spawn_ranks(_groups, 4, (buffer_size,), backend="gloo")


def _moved(rank, world, buffer_size):
    """``.to()`` of the wrapper moves module and buckets together; a move to another device type is refused while buckets exist."""
    model, oss = _sdp(_mlp(), buffer_size)
    model.to(torch.device("cpu"))
    model(_data(rank, 0)).sum().backward()
    oss.step()
    model.to(torch.device("cpu"), dtype=torch.float32)
    model.zero_grad()
    model(_data(rank, 1)).sum().backward()
    oss.step()


@pytest.mark.parametrize("buffer_size", [0, 2**16])
def test_sdp_to_same_device_keeps_training(buffer_size):
    spawn_ranks(_moved, 2, (buffer_size,), backend="gloo")


def _step_grid(rank, world, broadcast_buffers, accumulate, buffer_size, optimizer):
    opt_cls, opt_kw = (torch.optim.SGD, dict(lr=0.05, momentum=0.9)) if optimizer == "sgd" else (torch.optim.RMSprop, dict(lr=0.01))
    ref_net, net = _mlp(with_buffer=True), _mlp(with_buffer=True)
    ref = nn.parallel.DistributedDataParallel(ref_net, broadcast_buffers=broadcast_buffers)
    oss = OSS(net.parameters(), optim=opt_cls, **opt_kw)
    model = ShardedDataParallel(net, oss, broadcast_buffers=broadcast_buffers, reduce_buffer_size=buffer_size)
    ref_opt = opt_cls(ref.parameters(), **opt_kw)
    for step in range(4):
        for m, o in ((ref, ref_opt), (model, oss)):
            m.zero_grad()
            if accumulate:
                with m.no_sync():
                    m(_data(rank, 10 + step)).pow(2).mean().backward()
            m(_data(rank, step)).pow(2).mean().backward()
            o.step()
    for a, b in zip(ref_net.parameters(), net.parameters()):
        torch.testing.assert_close(b, a, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("broadcast_buffers,accumulate,buffer_size,optimizer", [(True, False, 0, "sgd"), (True, True, 2**16, "sgd"),
                                                                                (False, True, 0, "rmsprop"), (False, False, 2**16, "rmsprop")])
def test_sdp_step_configurations_match_ddp(broadcast_buffers, accumulate, buffer_size, optimizer):
    spawn_ranks(_step_grid, 2, (broadcast_buffers, accumulate, buffer_size, optimizer), backend="gloo")
