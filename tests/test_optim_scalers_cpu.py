"""AdaScale, ShardedGradScaler, LayerwiseGradientScaler on CPU (single process and gloo ranks)."""
import numpy as np
import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.nn.parallel import DistributedDataParallel as DDP
from torch.optim import SGD
from torch.optim.lr_scheduler import LambdaLR

from fairscale_b200.fair_dev.testing.golden_testing_data import adascale_test_data
from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.optim import OSS, AdaScale, AdaScaleWrapper, GradScaler, LayerwiseGradientScaler, ShardedGradScaler


def test_adascale_rejects_single_pass():
    with pytest.raises(RuntimeError):
        AdaScale(SGD(nn.Linear(2, 2).parameters(), lr=0.1))


@pytest.mark.parametrize("case", adascale_test_data)
@pytest.mark.parametrize("is_scaled_loss", [True, False])
def test_adascale_grad_accum_golden(case, is_scaled_loss):
    model = nn.Linear(2, 2, bias=True)
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=2, is_scaled_loss=is_scaled_loss)
    if "input" in case:
        data, gains = [case["input"]] * 2, [case["expected_gain"]] * 2
    else:
        data, gains = case["inputs"], [None, case["expected_gain"]]
    for pair, want in zip(data, gains):
        for x in pair:
            loss = model(torch.tensor(x)).sum()
            (loss / 2 if is_scaled_loss else loss).backward()
        if not is_scaled_loss:
            optim.scale_grad_by_num_grads_to_accum()
        if want is not None:
            assert np.allclose(optim.gain(), want), optim.gain()
            w, b = model.parameters()
            assert np.allclose(w.grad, case["expected_grad"]) and np.allclose(b.grad, case["expected_bias_grad"])
        optim.step()
        optim.zero_grad()


def test_adascale_lr_restored_scheduler_and_groups():
    model = nn.Linear(2, 2, bias=False)
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=2)
    sched = LambdaLR(optim, lr_lambda=lambda e: 0.5**e)
    for x in ([1.0, 0.0], [0.0, 1.0]):
        (model(torch.tensor(x)).sum() / 2).backward()
    before = model.weight.detach().clone()
    g = model.weight.grad.clone()
    optim.step()
    torch.testing.assert_close(model.weight, before - 0.1 * optim.gain(0) * g)
    assert optim.param_groups[0]["lr"] == 0.1
    sched.step()
    assert optim.param_groups[0]["lr"] == 0.05
    extra = nn.Linear(2, 2, bias=False)
    optim.add_param_group({"params": extra.parameters()})
    assert optim._state["grad_sqr_avg"].shape == (2,)
    assert isinstance(optim.state_dict(), dict)
    wrapped = AdaScaleWrapper(nn.Linear(2, 2).parameters(), num_gradients_to_accumulate=2, optim_cls=SGD, lr=0.3)
    assert wrapped.param_groups[0]["lr"] == 0.3 and wrapped.defaults["lr"] == 0.3


def _ddp_adascale(rank, world, case):
    model = nn.Linear(2, 2, bias=True)
    with torch.no_grad():
        model.weight.fill_(0.3)
        model.bias.fill_(0.1)
    ddp = DDP(model)
    optim = AdaScale(OSS(model.parameters(), SGD, lr=0.1))
    ddp(torch.tensor(case["input"][rank])).sum().backward()
    assert np.allclose(optim.gain(), case["expected_gain"]), optim.gain()
    optim.step()


@pytest.mark.parametrize("case", adascale_test_data[:5])
def test_adascale_ddp_two_ranks_golden(case):
    spawn_ranks(_ddp_adascale, 2, (case,), backend="gloo")


def test_grad_scaler_fp16_grads_and_sharded_cpu():
    model = nn.Linear(4, 4)
    opt = SGD(model.parameters(), lr=0.1)
    scaler = ShardedGradScaler(init_scale=8.0, growth_interval=1, device="cpu")
    loss = model(torch.ones(2, 4)).sum()
    scaler.scale(loss).backward()
    raw = model.weight.grad.clone()
    scaler.unscale_(opt)
    torch.testing.assert_close(model.weight.grad, raw / 8.0)
    before = model.weight.detach().clone()
    scaler.step(opt)
    scaler.update()
    assert not torch.equal(before, model.weight) and scaler.get_scale() == 16.0
    # overflow: step skipped, scale backs off
    opt.zero_grad()
    scaler.scale(model(torch.ones(2, 4)).sum()).backward()
    model.weight.grad[0, 0] = float("inf")
    before = model.weight.detach().clone()
    scaler.step(opt)
    scaler.update()
    assert torch.equal(before, model.weight) and scaler.get_scale() == 8.0
    assert isinstance(GradScaler(device="cpu", enabled=False).scale(loss), torch.Tensor)


def _sharded_scaler_rank(rank, world):
    model = nn.Linear(4, 4)
    opt = OSS(model.parameters(), SGD, lr=0.1)
    scaler = ShardedGradScaler(init_scale=4.0, device="cpu")
    scaler.scale(model(torch.ones(2, 4)).sum()).backward()
    if rank == 1:
        model.bias.grad[0] = float("nan")  # only one rank sees the overflow
    before = [p.detach().clone() for p in model.parameters()]
    scaler.step(opt)
    scaler.update()
    for b, p in zip(before, model.parameters()):
        assert torch.equal(b, p), "every rank must skip the step"
    assert scaler.get_scale() == 2.0


def test_sharded_grad_scaler_agrees_across_ranks():
    spawn_ranks(_sharded_scaler_rank, 2, (), backend="gloo")


def test_layerwise_gradient_scaler():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 2))
    ref = [p.detach().clone() for p in model.parameters()]
    x = torch.randn(3, 4, requires_grad=True)
    model(x).sum().backward()
    want = [p.grad.clone() for p in model.parameters()]
    model.zero_grad()
    scaler = LayerwiseGradientScaler(model, {"0": 1024.0, "2": 512.0, "4": 256.0}, growth_interval=1)
    scaler.scale()
    model(x).sum().backward()
    # parameter gradients of a layer carry that layer's factor until unscale()
    torch.testing.assert_close(model[4].weight.grad, want[4] * 256.0)
    torch.testing.assert_close(model[0].weight.grad, want[0] * 1024.0)
    scaler.unscale()
    for p, w in zip(model.parameters(), want):
        torch.testing.assert_close(p.grad, w)
    opt = SGD(model.parameters(), lr=0.1)
    scaler.step(opt)
    assert not torch.equal(ref[0], model[0].weight)
    assert [i.scaling_factor for i in scaler.get_layer_info() if i.scale_layer] == [2048.0, 1024.0, 512.0]
    model[2].weight.grad[0, 0] = float("inf")
    snap = model[0].weight.detach().clone()
    scaler.step(opt)
    assert torch.equal(snap, model[0].weight)
    assert [i.scaling_factor for i in scaler.get_layer_info() if i.scale_layer] == [4096.0, 512.0, 1024.0]  # only the layer that overflowed backs off


def _adascale_sequential(rank, world, mode):
    """Golden gain / mean weight of a 4-layer bias-free linear stack after two steps on orthogonal inputs, for AdaScale
    alone, AdaScale around OSS, AdaScaleWrapper building an OSS, and OSS around AdaScaleWrapper (values recorded by the
    reference's tests/optim/test_oss_adascale.py:95-130)."""
    from statistics import mean

    model = nn.Sequential(nn.Linear(2, 3, bias=False), nn.Linear(3, 4, bias=False), nn.Linear(4, 5, bias=False), nn.Linear(5, 6, bias=False))
    with torch.no_grad():
        for layer, n in zip(model, (6, 12, 20, 30)):
            layer.weight.copy_(torch.arange(n, dtype=torch.float32).reshape(layer.weight.shape) / mean(range(n)))
    ddp = DDP(model)
    if mode == "ada-oss":
        optim = AdaScale(OSS(ddp.parameters(), SGD, lr=0.1))
    elif mode == "wrapper-oss":
        optim = AdaScaleWrapper(ddp.parameters(), optim_cls=OSS, optim=SGD, lr=0.1)
    elif mode == "oss-wrapper":
        optim = OSS(ddp.parameters(), AdaScaleWrapper, optim_cls=SGD, lr=0.1)
    else:
        optim = AdaScale(SGD(ddp.parameters(), lr=0.1))
    for inputs in ([[1.0, 0], [0, 1.0]], [[0, 1.0], [1.0, 0]]):
        ddp(torch.tensor(inputs[rank])).sum().backward()
        optim.step()
        optim.zero_grad()
    mean_weight = mean(layer.weight.data.mean().item() for layer in model)
    if mode == "oss-wrapper":  # every rank scales its own shard: numerically a different algorithm, only the weights are pinned
        assert np.allclose(mean_weight, 94.93386840820312, rtol=1e-5), mean_weight
    else:
        assert np.allclose(optim.gain(), 1.0335265132125744, rtol=1e-6), optim.gain()
        assert np.allclose(mean_weight, 52.92657661437988, rtol=1e-5), mean_weight


@pytest.mark.parametrize("mode", ["none", "ada-oss", "wrapper-oss", "oss-wrapper"])
def test_adascale_with_oss_sequential_golden(mode):
    spawn_ranks(_adascale_sequential, 2, (mode,), backend="gloo")
