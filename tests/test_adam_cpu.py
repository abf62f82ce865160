"""The Adam front-end on CPU tensors (the PyTorch restatement of the kernel math): parity with torch.optim.Adam / AdamW,
the four precision modes, state-dict round trip with ``optim_scale``, overflow handling of scaled fp16 moments."""
import copy

import pytest
import torch
from torch import nn

from fairscale_b200.optim import Adam
from fairscale_b200.optim.adam import Precision


def _model(dtype=torch.float32):
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(6, 9), nn.Tanh(), nn.Linear(9, 3)).to(dtype)


def _grads(model, step):
    g = torch.Generator().manual_seed(step)
    x = torch.randn(5, 6, generator=g).to(next(model.parameters()).dtype)
    model.zero_grad()
    model(x).float().pow(2).mean().backward()


@pytest.mark.parametrize("wd,decoupled", [(0.0, False), (0.1, True)])
def test_full_precision_matches_torch(wd, decoupled):
    a, b = _model(), _model()
    ours = Adam(a.parameters(), lr=1e-2, weight_decay=wd, decoupled_weight_decay=decoupled)
    ref_cls = torch.optim.AdamW if decoupled else torch.optim.Adam
    ref = ref_cls(b.parameters(), lr=1e-2, weight_decay=wd)
    for s in range(5):
        _grads(a, s)
        _grads(b, s)
        ours.step()
        ref.step()
    # the kernel folds both bias corrections into the step size (eps is added to the uncorrected sqrt(v), as in the
    # reference's fused Adam), torch corrects v first: the updates differ by O(eps)
    for p, q in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(p, q, atol=1e-5, rtol=1e-4)


def test_coupled_weight_decay_follows_the_fused_kernel_formula():
    """With ``weight_decay`` (not decoupled) the decay term joins the normalised update, ``p -= step * (m / denom + wd * p)``,
    as in the reference's kernel (fused_adam_cuda_kernel.cu:108-129), not torch's L2-into-the-gradient form."""
    a = _model()
    p0 = [p.detach().clone() for p in a.parameters()]
    opt = Adam(a.parameters(), lr=1e-2, weight_decay=0.1)
    _grads(a, 0)
    g = [p.grad.clone() for p in a.parameters()]
    opt.step()
    step = 1e-2 * (1 - 0.999) ** 0.5 / (1 - 0.9)
    for p, q, gr in zip(a.parameters(), p0, g):
        m, v = 0.1 * gr, 0.001 * gr * gr
        torch.testing.assert_close(p.detach(), q - step * (m / (v.sqrt() + 1e-8) + 0.1 * q), atol=1e-6, rtol=1e-5)


def test_eps_inside_sqrt_and_no_bias_correction():
    a = _model()
    p0 = [p.detach().clone() for p in a.parameters()]
    opt = Adam(a.parameters(), lr=1e-2, eps=1e-4, eps_inside_sqrt=True, bias_correction=False)
    _grads(a, 0)
    g = [p.grad.clone() for p in a.parameters()]
    opt.step()
    for p, q, gr in zip(a.parameters(), p0, g):
        m, v = 0.1 * gr, 0.001 * gr * gr
        torch.testing.assert_close(p.detach(), q - 1e-2 * m / torch.sqrt(v + 1e-4), atol=1e-6, rtol=1e-5)
    with pytest.raises(RuntimeError):
        Adam(a.parameters(), amsgrad=True)


def test_mixed_precision_keeps_fp32_masters():
    a, b = _model(torch.bfloat16), _model()
    for p, q in zip(a.parameters(), b.parameters()):
        q.data.copy_(p.data.float())  # same starting point: the bf16-rounded weights
    ours = Adam(a.parameters(), lr=1e-2)
    assert ours.precision is Precision.MIXED_PRECISION and ours.mixed_precision
    ref = torch.optim.Adam(b.parameters(), lr=1e-2)
    for s in range(4):
        _grads(a, s)
        for p, q in zip(a.parameters(), b.parameters()):
            q.grad = p.grad.float()
        ours.step()
        ref.step()
    masters = [m for grp in ours.fp32_param_groups for m in grp["params"]]
    for m, p, q in zip(masters, a.parameters(), b.parameters()):
        assert m.dtype == torch.float32
        torch.testing.assert_close(m, q, atol=1e-5, rtol=1e-4)       # the master follows fp32 Adam
        torch.testing.assert_close(p.float(), m.bfloat16().float())   # the model holds its rounding


def test_memory_efficient_mode_updates_low_precision_params_with_fp32_moments():
    a = _model(torch.bfloat16)
    opt = Adam(a.parameters(), lr=1e-2, precision=Precision.MEMORY_EFFICIENT_MIXED_PRECISION)
    before = [p.detach().clone() for p in a.parameters()]
    _grads(a, 0)
    opt.step()
    assert not opt.fp32_param_groups
    for p, q in zip(a.parameters(), before):
        assert p.dtype == torch.bfloat16 and not torch.equal(p, q)
        assert opt.state[p]["exp_avg"].dtype == torch.float32


def test_pure_fp16_scaled_moments_state_dict_and_overflow():
    a = _model(torch.float16)
    opt = Adam(a.parameters(), lr=1e-3, precision=Precision.PURE_FP16)
    assert opt._optim_scale == 2.0**16
    _grads(a, 0)
    opt.step()
    p = next(a.parameters())
    assert opt.state[p]["exp_avg"].dtype == torch.float16
    # moments are stored times optim_scale
    torch.testing.assert_close(opt.state[p]["exp_avg"].float() / opt._optim_scale, 0.1 * p.grad.float(), atol=1e-4, rtol=2e-2)
    sd = copy.deepcopy(opt.state_dict())
    assert sd["optim_scale"] == 2.0**16
    b = _model(torch.float16)
    opt2 = Adam(b.parameters(), lr=1e-3, precision=Precision.PURE_FP16)
    sd["optim_scale"] = 2.0**10
    opt2.load_state_dict(sd)
    assert opt2._optim_scale == 2.0**10 and opt2.state[next(b.parameters())]["exp_avg"].dtype == torch.float16
    # a huge gradient overflows the scaled fp16 moments: the scale is halved and the moments restart from zero
    _grads(a, 1)
    for q in a.parameters():
        q.grad.fill_(60000.0)
    scale = opt._optim_scale
    opt.step()
    assert opt._optim_scale == scale / 2
    assert all(torch.count_nonzero(opt.state[q]["exp_avg"]) == 0 for q in a.parameters())
