"""More of the Adam front-end on CPU tensors (cases of the reference's tests/optim/test_adam.py that need no GPU): state
dicts of the four precision modes reproduce the next step, the moment scale grows back and refuses to fall below one,
master copies, argument checks, precision / dtype mismatches, parameter groups, closures, parameters without gradients,
sparse gradients, the folded-in unscale factor and skip flag, extra low-precision copies, and training under a GradScaler."""
import copy

import pytest
import torch
from torch import nn

from fairscale_b200.optim import Adam, GradScaler
from fairscale_b200.optim.adam import Precision


def _params(dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    weight = torch.randn(10, 5, generator=g).to(dtype).requires_grad_()
    bias = torch.randn(10, generator=g).to(dtype).requires_grad_()
    x = torch.randn(5, generator=g).to(dtype)
    return weight, bias, x


def _backward(weight, bias, x):
    for p in (weight, bias):
        p.grad = None
    loss = (weight.mv(x) + bias).float().pow(2).sum()
    loss.backward()
    return float(loss)


MODES = [(torch.float32, Precision.FULL_PRECISION), (torch.float16, Precision.MIXED_PRECISION), (torch.bfloat16, Precision.MIXED_PRECISION),
         (torch.bfloat16, Precision.MEMORY_EFFICIENT_MIXED_PRECISION), (torch.float16, Precision.PURE_FP16)]


@pytest.mark.parametrize("dtype,precision", MODES)
def test_loss_goes_down_in_every_mode(dtype, precision):
    weight, bias, x = _params(dtype)
    opt = Adam([weight, bias], lr=1e-2, precision=precision)
    first = _backward(weight, bias, x)
    for _ in range(8):
        opt.step()
        last = _backward(weight, bias, x)
    assert last < first
    state_dtype = torch.float16 if precision is Precision.PURE_FP16 else torch.float32
    assert opt.state[weight]["exp_avg"].dtype == state_dtype and opt.state[weight]["exp_avg_sq"].dtype == state_dtype
    assert weight.dtype == dtype and opt.state[weight]["step"] == 8


@pytest.mark.parametrize("dtype,precision", MODES)
def test_state_dict_reproduces_the_next_step(dtype, precision):
    weight, bias, x = _params(dtype)
    opt = Adam([weight, bias], lr=1e-2, precision=precision)
    for _ in range(3):
        _backward(weight, bias, x)
        opt.step()
    saved = copy.deepcopy(opt.state_dict())
    assert saved["optim_scale"] == opt._optim_scale and (precision is Precision.PURE_FP16 or saved["optim_scale"] == 1.0)

    w2, b2 = weight.detach().clone().requires_grad_(), bias.detach().clone().requires_grad_()
    other = Adam([w2, b2], lr=1e-2, precision=precision)
    if precision is Precision.MIXED_PRECISION:
        # the master copies are part of the run: carry them over as a user restoring a checkpoint would
        for src, dst in zip(opt.fp32_param_groups[0]["params"], other.fp32_param_groups[0]["params"]):
            dst.data.copy_(src.data)
    other.load_state_dict(saved)
    assert other.state[w2]["step"] == 3 and other.state[w2]["exp_avg"].dtype == opt.state[weight]["exp_avg"].dtype
    _backward(weight, bias, x)
    _backward(w2, b2, x)
    opt.step()
    other.step()
    assert torch.equal(weight, w2) and torch.equal(bias, b2)
    assert torch.equal(opt.state[weight]["exp_avg_sq"], other.state[w2]["exp_avg_sq"])


def test_moment_scale_grows_back_and_is_capped():
    weight, bias, x = _params(torch.float16)
    opt = Adam([weight, bias], lr=1e-3, precision=Precision.PURE_FP16)
    opt._optim_scale_update_freq = 1
    opt._optim_scale = 2.0**15
    x = x * 0.01  # gradients small enough for the scaled fp16 moments
    with torch.no_grad():
        weight.mul_(0.01)
        bias.mul_(0.01)
    _backward(weight, bias, x)
    opt.step()
    assert opt._optim_scale == 2.0**16
    _backward(weight, bias, x)
    opt.step()
    assert opt._optim_scale == 2.0**16  # never above the starting scale


def test_moment_scale_below_one_means_exploding_gradients():
    weight = torch.tensor([[float("inf")]]).half().requires_grad_()
    opt = Adam([weight], lr=1e-3, precision=Precision.PURE_FP16)
    opt._optim_scale = 1.0
    (weight.mv(torch.tensor([1.0]).half())).float().pow(2).sum().backward()
    with pytest.raises(RuntimeError, match="scale"):
        opt.step()


def test_master_copies_mirror_the_parameters():
    weight, bias, _ = _params(torch.float16)
    opt = Adam([weight, bias], lr=1e-3)
    assert opt.precision is Precision.MIXED_PRECISION
    for masters, group in zip(opt.fp32_param_groups, opt.param_groups):
        for m, p in zip(masters["params"], group["params"]):
            assert m.dtype == torch.float32 and p.dtype == torch.float16 and torch.equal(m.data, p.data.float())
    with torch.no_grad():
        weight.add_(1.0)
    opt._build_fp32_params()  # rebuilt from the current values
    assert torch.equal(opt.fp32_param_groups[0]["params"][0].data, weight.data.float())


@pytest.mark.parametrize("kwargs", [dict(betas=(1.0, 0.0)), dict(betas=(0.9, 1.5)), dict(betas=(-0.1, 0.9)), dict(weight_decay=-1),
                                    dict(lr=-1e-3), dict(eps=-1e-8)])
def test_arguments_out_of_range_are_refused(kwargs):
    weight, bias, _ = _params(torch.float32)
    with pytest.raises(ValueError):
        Adam([weight, bias], **{"lr": 1e-2, **kwargs})


def test_amsgrad_is_refused():
    weight, bias, _ = _params(torch.float32)
    with pytest.raises(RuntimeError, match="AMSGrad"):
        Adam([weight, bias], lr=1e-2, amsgrad=True)


@pytest.mark.parametrize("precision", [Precision.MIXED_PRECISION, Precision.MEMORY_EFFICIENT_MIXED_PRECISION, Precision.PURE_FP16])
def test_low_precision_modes_want_low_precision_parameters(precision):
    weight, bias, _ = _params(torch.float32)
    with pytest.raises(AssertionError):
        Adam([weight, bias], lr=1e-2, precision=precision)


def test_parameter_groups_keep_their_own_settings():
    weight, bias, x = _params(torch.float32)
    w0, b0 = weight.detach().clone(), bias.detach().clone()
    opt = Adam([{"params": [weight], "lr": 1e-1}, {"params": [bias], "lr": 0.0, "weight_decay": 0.0}], lr=1e-3)
    assert opt.param_groups[0]["lr"] == 1e-1 and opt.param_groups[1]["lr"] == 0.0
    _backward(weight, bias, x)
    opt.step()
    assert not torch.equal(weight, w0) and torch.equal(bias, b0)  # a zero rate moves nothing
    # the first step of Adam moves every weight by about the learning rate
    assert float((weight.detach() - w0).abs().max()) == pytest.approx(1e-1, rel=1e-3)
    assert opt.group_of(bias) is opt.param_groups[1] and opt.group_of(torch.zeros(1)) is None


def test_closure_and_parameters_without_gradients():
    weight, bias, x = _params(torch.float32)
    unused = torch.zeros(3, requires_grad=True)
    opt = Adam([weight, bias, unused], lr=1e-2)
    calls = []

    def closure():
        calls.append(1)
        return _backward(weight, bias, x)

    loss = opt.step(closure)
    assert calls == [1] and loss == pytest.approx(_backward(weight, bias, x), rel=0.2)
    assert unused not in opt.state and torch.count_nonzero(unused) == 0
    assert opt.supports_memory_efficient_fp16 and not opt._step_supports_amp_scaling


def test_sparse_gradients_are_refused():
    emb = nn.Embedding(10, 4, sparse=True)
    opt = Adam(emb.parameters(), lr=1e-2)
    emb(torch.tensor([1, 2])).sum().backward()
    with pytest.raises(RuntimeError, match="sparse"):
        opt.step()


def test_unscale_factor_skip_flag_and_extra_copies():
    weight, bias, x = _params(torch.float32)
    w2, b2 = weight.detach().clone().requires_grad_(), bias.detach().clone().requires_grad_()
    plain, folded = Adam([weight, bias], lr=1e-2), Adam([w2, b2], lr=1e-2)
    _backward(weight, bias, x)
    _backward(w2, b2, x)
    for p in (w2, b2):
        p.grad.mul_(128.0)  # as a loss scaler leaves them
    folded.inv_scale = torch.tensor([1.0 / 128.0])
    copy16 = torch.zeros_like(w2, dtype=torch.bfloat16)
    folded.param_copies[w2] = copy16
    plain.step()
    folded.step()
    torch.testing.assert_close(w2, weight, atol=1e-7, rtol=1e-6)
    assert torch.equal(copy16, w2.detach().bfloat16())  # the copy a wrapper asked for was written by the same pass
    # the skip flag leaves parameters and moments alone
    before, m_before = w2.detach().clone(), folded.state[w2]["exp_avg"].clone()
    folded.noop_flag = torch.tensor([1])
    _backward(w2, b2, x)
    folded.step()
    assert torch.equal(w2, before) and torch.equal(folded.state[w2]["exp_avg"], m_before)
    folded.noop_flag.zero_()
    folded.inv_scale = None
    folded.step()
    assert not torch.equal(w2, before)


def test_training_under_a_grad_scaler_in_pure_fp16():
    weight, bias, x = _params(torch.float16)
    opt = Adam([weight, bias], lr=1e-3, precision=Precision.PURE_FP16)
    scaler = GradScaler(device="cpu", init_scale=2.0**8)
    first = last = None
    for i in range(5):
        opt.zero_grad()
        loss = (weight.mv(x) + bias).float().pow(2).sum()
        first = float(loss) if i == 0 else first
        last = float(loss)
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
    assert last < first
