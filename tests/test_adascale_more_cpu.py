"""AdaScale beyond the basic gains (cases of the reference's tests/optim/test_single_node_adascale.py and
test_ddp_adascale.py, on CPU and gloo): resuming from a checkpoint reproduces the run, learning-rate schedulers see the
unscaled rate, parameter groups added before and after a step have their own gains, the accumulation count can change
between steps, de-biased averages, gradients are left alone by the hooks, a scale other than the number of passes,
releasing the hooks, accumulation under ``no_sync`` on two ranks and the correlation of the ranks' gradients."""
import gc
import weakref

import numpy as np
import pytest
import torch
import torch.distributed as dist
from torch import Tensor
from torch.nn import Linear, Sequential
from torch.nn.parallel import DistributedDataParallel as DDP
from torch.optim import SGD
from torch.optim.lr_scheduler import LambdaLR

from fairscale_b200.fair_dev.testing.golden_testing_data import adascale_test_data, corr_mean_test_data
from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.fair_dev.testing.testing_memory import find_tensor_by_shape
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP
from fairscale_b200.nn.data_parallel import ShardedDataParallel as SDP
from fairscale_b200.optim import OSS, AdaScale


def test_loss_accumulation_is_not_gradient_accumulation():
    """Summing two losses and calling backward once is one pass as far as AdaScale can tell: it refuses to report a gain."""
    model = Linear(2, 2, bias=False)
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=3)
    (model(Tensor([0.0, 1.0])).sum() + model(Tensor([1.0, 0.0])).sum()).backward()
    with pytest.raises((AssertionError, RuntimeError)):
        optim.step()  # one backward where three were announced


def test_resuming_from_a_checkpoint_reproduces_the_run(tmp_path):
    accum, width = 3, 5

    def fresh():
        torch.manual_seed(7)
        model = Linear(width, 2, bias=False)
        return model, AdaScale(SGD(model.parameters(), lr=0.1, momentum=0.9), num_gradients_to_accumulate=accum)

    def run(model, optim, data=None):
        used, out = [], None
        for step in range(6):
            for i in range(accum):
                x = torch.rand(width) if data is None else data[step * accum + i]
                used.append(x)
                out = model(x)
                out.sum().backward()
            optim.step()
            optim.zero_grad()
        return float(out.sum()), used

    model, optim = fresh()
    torch.manual_seed(11)
    run(model, optim)
    torch.save({"model": model.state_dict(), "optim": optim.state_dict()}, tmp_path / "ckpt.pt")
    want_out, replay = run(model, optim)
    want_gain = optim.gain()

    model, optim = fresh()
    ckpt = torch.load(tmp_path / "ckpt.pt", weights_only=False)
    model.load_state_dict(ckpt["model"])
    optim.load_state_dict(ckpt["optim"])
    got_out, _ = run(model, optim, replay)
    assert np.allclose(got_out, want_out) and np.allclose(optim.gain(), want_gain)


def test_scheduler_sees_the_plain_learning_rate():
    accum = 3
    model = Linear(2, 2, bias=False)
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=accum)
    scheduler = LambdaLR(optim, lr_lambda=lambda epoch: 1 / 10**epoch)
    torch.manual_seed(0)
    for epoch in range(3):
        for _ in range(10):
            for _ in range(accum):
                model(torch.rand(2)).sum().backward()
            assert optim.gain() <= 3
            optim.step()
            optim.zero_grad()
            assert np.allclose(optim.param_groups[0]["lr"], 0.1 / 10**epoch)  # the gain was applied for the step only
        scheduler.step()
        assert np.allclose(optim.param_groups[0]["lr"], 0.1 / 10 ** (epoch + 1))


def _filled(linear, values, bias):
    with torch.no_grad():
        linear.weight.copy_(Tensor(values).reshape(linear.weight.shape))
        linear.bias.fill_(bias)
    return linear


@pytest.mark.parametrize("debias_ewma", [True, False])
@pytest.mark.parametrize("is_scaled_loss", [True, False])
def test_parameter_groups_added_before_and_after_a_step(debias_ewma, is_scaled_loss):
    accum = 2
    first = _filled(Linear(2, 2), [1.0, 2.0, 3.0, 4.0], 0.1)
    optim = AdaScale(SGD(first.parameters(), lr=0.1), num_gradients_to_accumulate=accum, is_scaled_loss=is_scaled_loss, debias_ewma=debias_ewma)
    assert len(optim._hook_handles) == 2
    second = _filled(Linear(2, 3), [1.0, 2.0, 3.0, 4.0, 5.0, 6.0], 0.2)
    optim.add_param_group({"params": second.parameters()})
    assert len(optim._hook_handles) == 4

    def two_passes(model):
        for x in ([1.0, 2.0], [3.0, 4.0]):
            loss = model(Tensor(x)).sum()
            (loss / accum if is_scaled_loss else loss).backward()
        if not is_scaled_loss:
            optim.scale_grad_by_num_grads_to_accum()

    two_passes(Sequential(first, second))
    # the first step: de-biasing changes nothing yet
    assert np.allclose(optim.gain(), 1.1440223454935758), optim.gain()
    assert np.allclose(optim.gain(0), 1.1428571428571428), optim.gain(0)
    assert np.allclose(optim.gain(1), 1.1471258476157762), optim.gain(1)
    optim.step()
    optim.zero_grad()

    third = _filled(Linear(3, 4), [1.0, 2.0, 3.0, 4.0, 5.0, 6.0] * 2, 0.2)
    optim.add_param_group({"params": third.parameters()})
    assert len(optim._hook_handles) == 6
    two_passes(Sequential(first, second, third))
    assert np.allclose(optim.gain(), 1.1382937715383077 if debias_ewma else 1.1391959826562015), optim.gain()
    assert np.allclose(optim.gain(0), 1.142857206008338 if debias_ewma else 1.142857206006931), optim.gain(0)
    assert np.allclose(optim.gain(1), 1.1116875516387468 if debias_ewma else 1.1116906378271827), optim.gain(1)
    assert np.allclose(optim.gain(2), 1.0749164095196344), optim.gain(2)  # first step of this group either way
    optim.step()
    optim.zero_grad()


@pytest.mark.parametrize("accum,want", [(3, 2.141385737279438), (6, 2.9927880097754036), (9, 3.4461759591877312)])
@pytest.mark.parametrize("is_scaled_loss", [True, False])
def test_accumulation_count_changed_between_steps(accum, want, is_scaled_loss):
    model = Linear(2, 2, bias=False)
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=2, is_scaled_loss=is_scaled_loss)
    for x in ([0.0, 1.0], [1.0, 0.0]):
        loss = model(Tensor(x)).sum()
        (loss / 2 if is_scaled_loss else loss).backward()
    if not is_scaled_loss:
        optim.scale_grad_by_num_grads_to_accum()
    assert np.allclose(optim.gain(), 2.0)
    optim.step()
    optim.zero_grad()

    optim.set_scale(float(accum))
    optim.set_num_gradients_to_accumulate(accum)
    for _ in range(accum):
        loss = model(Tensor([0.0, 1.0])).sum() / accum
        (loss / accum if is_scaled_loss else loss).backward()
    if not is_scaled_loss:
        optim.scale_grad_by_num_grads_to_accum()
    assert np.allclose(optim.gain(), want), optim.gain()
    optim.step()
    optim.zero_grad()


def test_debiased_averages_give_the_exact_gain_from_the_first_step():
    model = Linear(2, 2, bias=False)
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=2, debias_ewma=True)
    for _ in range(4):
        model(Tensor([0.0, 1.0])).sum().backward()
        model(Tensor([1.0, 0.0])).sum().backward()
        assert np.allclose(optim.gain(), 2.0), optim.gain()
        optim.step()
        optim.zero_grad()


def test_hooks_leave_the_gradients_alone():
    model = Linear(2, 2, bias=False)
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=2)
    model(Tensor([0.0, 1.0])).sum().backward()
    assert np.allclose(model.weight.grad.numpy(), [[0.0, 1.0], [0.0, 1.0]])
    model(Tensor([0.0, 1.0])).sum().backward()
    assert np.allclose(model.weight.grad.numpy(), [[0.0, 2.0], [0.0, 2.0]])
    assert np.allclose(optim.gain(), 1.0000002499999376), optim.gain()  # identical passes: no gain to be had
    optim.step()
    assert np.allclose(model.weight.grad.numpy(), [[0.0, 2.0], [0.0, 2.0]])
    optim.zero_grad()
    assert model.weight.grad is None or np.allclose(model.weight.grad.numpy(), 0.0)


@pytest.mark.parametrize("scale,want", [(None, 4.0), (4.0 / 3, 4.0 / 3), (2.0, 2.0), (4.0, 4.0)])
def test_scale_other_than_the_number_of_passes(scale, want):
    model = Linear(4, 2, bias=False)
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=4, scale=scale)
    for i in range(4):  # orthogonal inputs: the gain reaches the scale
        model(torch.eye(4)[i]).sum().backward()
    assert np.allclose(optim.gain(), want), optim.gain()


def test_unhook_releases_the_parameters():
    model = Linear(123, 457, bias=False)  # a shape nothing else has
    ref = weakref.ref(model.weight)
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=2)
    assert find_tensor_by_shape((457, 123))
    optim.unhook()
    assert len(optim._hook_handles) == 0
    del model, optim
    gc.collect()
    assert ref() is None and not find_tensor_by_shape((457, 123))


def test_smoothing_factor_given_or_derived():
    model = Linear(1, 1)
    assert AdaScale(SGD(model.parameters(), lr=0.1), smoothing=0.12345, num_gradients_to_accumulate=3)._smoothing == 0.12345
    derived = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=3)
    assert 0.0 < derived.smoothing < 1.0
    derived.set_num_gradients_to_accumulate(6)
    assert derived.smoothing > 0.0


# ------------------------------------------------------------------------------------------------ two ranks
def _wrappers(rank, world, wrapper, case):
    model = Linear(2, 2)
    if wrapper == "ddp":
        model = DDP(model)
        optim = AdaScale(SGD(model.parameters(), lr=0.1))
    elif wrapper == "sdp":
        optim = AdaScale(OSS(model.parameters(), SGD, lr=0.1))
        model = SDP(model, sharded_optimizer=optim)
    else:
        model = FSDP(model, flatten_parameters=False)  # AdaScale after the wrapper: it hooks the sharded parameters
        optim = AdaScale(SGD(model.parameters(), lr=0.1))
    batches = [case["input"]] if "input" in case else case["inputs"]
    for i, batch in enumerate(batches):
        model(Tensor(batch[rank])).sum().backward()
        if i == len(batches) - 1 and wrapper == "ddp":
            assert np.allclose(optim.gain(), case["expected_gain"]), optim.gain()
            w, b = model.parameters()
            assert np.allclose(w.grad, case["expected_grad"]) and np.allclose(b.grad, case["expected_bias_grad"])
        assert 1.0 <= optim.gain() <= 2.0 + 1e-6
        optim.step()
        optim.zero_grad()


@pytest.mark.parametrize("case", [adascale_test_data[0], adascale_test_data[3], adascale_test_data[-1]], ids=["orthogonal", "generic", "two_steps"])
def test_two_ranks_under_ddp_reach_the_golden_gain(case):
    spawn_ranks(_wrappers, 2, ("ddp", case), backend="gloo")


@pytest.mark.parametrize("wrapper", ["sdp", "fsdp"])
def test_two_ranks_under_the_sharded_wrappers_step(wrapper):
    spawn_ranks(_wrappers, 2, (wrapper, adascale_test_data[0]), backend="gloo")


def _accumulate_under_no_sync(rank, world):
    model = DDP(Linear(4, 2, bias=False))
    optim = AdaScale(SGD(model.parameters(), lr=0.1), num_gradients_to_accumulate=2)
    with model.no_sync():
        model(torch.eye(4)[rank]).sum().backward()
    model(torch.eye(4)[rank + 2]).sum().backward()
    assert np.allclose(optim.gain(), 4.0), optim.gain()  # four orthogonal gradients over two ranks and two passes
    optim.step()
    optim.zero_grad()


def test_accumulation_under_no_sync_counts_every_rank_and_pass():
    spawn_ranks(_accumulate_under_no_sync, 2, (), backend="gloo")


def _gradient_correlation(rank, world, case):
    model = DDP(Linear(3, 1, bias=False))
    optim = AdaScale(SGD(model.parameters(), lr=0.1))
    corr, last = [], None
    for i, batch in enumerate(case["inputs"]):
        with model.no_sync():  # local gradients stay local: that is what the correlation is about
            model(Tensor(batch[rank])).sum().backward()
            corr.append(float(optim._compute_intra_grad_corr_mean()))
        for p in model.parameters():
            dist.all_reduce(p.grad)
            p.grad.div_(world)
        grad = optim._gather_flat_grad().clone()
        assert np.allclose(grad, case["expected_grad"][i])
        optim.step()
        if last is not None:
            cos = float(torch.dot(grad, last) / (grad.norm() * last.norm()))
            assert np.allclose(cos, case["expected_cos_similarity"][i], atol=1e-4), cos
        last = grad
        optim.zero_grad()
    assert np.allclose(corr, case["expected_corr"], atol=1e-6), corr


def test_correlation_of_the_ranks_gradients():
    spawn_ranks(_gradient_correlation, 2, (corr_mean_test_data[0],), backend="gloo")
