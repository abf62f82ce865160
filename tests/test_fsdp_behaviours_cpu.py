"""Remaining single behaviours of the reference's tests/nn/data_parallel/test_fsdp.py, on gloo ranks with bf16 as the
low-precision type: which dtype the wrapped module sees for its input, parameters, buffers and loss in every precision
setting (and which dtype the gradients are reduced in), weights changed in place after wrapping, the reduce-scatter group,
output hooks after a local state dict was loaded, hook registration during forward, parameter names before and after
wrapping and inside ``summon_full_params``, ``reset_parameters``, gradient clipping with several norms, optimizer steps
delayed past the next forward, evaluation with and without ``no_grad``."""
from math import inf
from unittest import mock

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import DeviceAndTypeCheckModule, objects_are_equal, spawn_ranks
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP
from fairscale_b200.parallel import comm

CPU = torch.device("cpu")
LOW = torch.bfloat16


class _Shared(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.embed_tokens = nn.Embedding(23, 16)
        self.body = nn.Sequential(nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 16))
        self.output_proj = nn.Linear(16, 23, bias=False)
        self.output_proj.weight = self.embed_tokens.weight
        self.vocab_bias = nn.Parameter(torch.zeros(23))

    def forward(self, tokens):
        return self.output_proj(self.body(self.embed_tokens(tokens))) + self.vocab_bias


def _tokens(rank=0):
    return torch.arange(12).view(3, 4) + rank


def _wrapped(**config):
    return FSDP(_Shared(), compute_device=CPU, **config)


def _train(model, rank, steps=1):
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    for _ in range(steps):
        opt.zero_grad()
        model(_tokens(rank)).float().pow(2).mean().backward()
        opt.step()
    return opt


# ------------------------------------------------------------------------------------------------ dtypes seen by the module
def _dtypes(rank, world, config, autocast, want_input, want_param, want_loss, want_reduce, want_buffer):
    module = DeviceAndTypeCheckModule(expected_input_dtype=want_input, expected_param_dtype=want_param, expected_loss_dtype=want_loss,
                                      expected_buffer_dtype=want_buffer)
    cfg = dict(config, compute_device=CPU)
    if cfg.get("mixed_precision") and "compute_dtype" not in cfg:
        cfg["compute_dtype"] = LOW
    model = FSDP(module, **cfg)
    seen = []
    comm.add_listener(lambda kind, group, out, inp: seen.append((kind, inp.dtype if torch.is_tensor(inp) else inp[0].dtype)) if kind == "reduce_scatter" else None)
    x = torch.rand(8, 5)
    with torch.autocast("cpu", dtype=LOW, enabled=autocast):
        loss = model(x)
    loss.backward()
    assert seen and all(dtype == want_reduce for _, dtype in seen), (seen, want_reduce)


@pytest.mark.parametrize("config,autocast,want_input,want_param,want_loss,want_reduce,want_buffer", [
    (dict(mixed_precision=False), False, torch.float32, torch.float32, torch.float32, torch.float32, torch.float32),
    (dict(mixed_precision=True), False, LOW, LOW, LOW, LOW, LOW),
    # under autocast on a CPU the final sum stays in the low-precision type (CUDA autocast promotes it): not checked there
    (dict(mixed_precision=True), True, LOW, LOW, None, LOW, LOW),
    (dict(mixed_precision=True, buffer_dtype=torch.float32), True, LOW, LOW, torch.float32, LOW, torch.float32),
    # inputs are cast to the compute type (the reference always casts them to half precision)
    (dict(mixed_precision=True, compute_dtype=torch.float32), True, torch.float32, torch.float32, None, torch.float32, torch.float32),
    (dict(mixed_precision=True, fp32_reduce_scatter=True), False, LOW, LOW, LOW, torch.float32, LOW),
    (dict(mixed_precision=True, fp32_reduce_scatter=True), True, LOW, LOW, None, torch.float32, LOW),
], ids=["all_fp32", "mixed", "mixed_autocast", "mixed_autocast_fp32_buffers", "mixed_autocast_fp32_compute", "fp32_reduce_scatter",
        "fp32_reduce_scatter_autocast"])
def test_dtypes_seen_by_the_wrapped_module(config, autocast, want_input, want_param, want_loss, want_reduce, want_buffer):
    spawn_ranks(_dtypes, 2, (config, autocast, want_input, want_param, want_loss, want_reduce, want_buffer), backend="gloo")


def _needs_mixed(rank, world):
    with pytest.raises(ValueError):
        FSDP(nn.Linear(2, 2), fp32_reduce_scatter=True, compute_device=CPU)


def test_fp32_reduce_scatter_needs_mixed_precision():
    spawn_ranks(_needs_mixed, 1, (), backend="gloo")


# ------------------------------------------------------------------------------------------------ single behaviours
def _single_behaviours(rank, world):
    # a weight changed in place after wrapping is what the next forward uses
    before = _wrapped(mixed_precision=True, compute_dtype=LOW).eval()(_tokens())
    model = _wrapped(mixed_precision=True, compute_dtype=LOW).eval()
    nn.init.normal_(next(model.parameters()).data)
    assert not objects_are_equal(before, model(_tokens()))

    # the reduce-scatter group spans the same ranks as the main group, for nested instances too
    nested = FSDP(nn.Sequential(FSDP(nn.Linear(4, 4), compute_device=CPU), nn.Linear(4, 4)), compute_device=CPU)
    for m in nested.modules():
        if isinstance(m, FSDP):
            assert dist.get_world_size(m.process_group_reduce_scatter) == m.world_size == world

    # hooks on the output: one pre-backward hook, still in place after backward and after a local state dict round trip
    model = _wrapped()
    _train(model, rank, 2)
    model.load_local_state_dict(model.local_state_dict())
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    opt.zero_grad()
    out = model(_tokens(rank))
    assert len(out._backward_hooks) == 1
    out.float().pow(2).mean().backward()
    assert len(out._backward_hooks) == 1
    opt.step()

    # both kinds of hooks are registered during forward
    model = _wrapped()
    with mock.patch.object(model, "_register_post_backward_hooks", return_value=None) as post:
        with mock.patch.object(model, "_register_pre_backward_hooks", side_effect=lambda outputs: outputs) as pre:
            assert not post.called and not pre.called
            model(_tokens(rank))
            assert post.called and pre.called

    # reset_parameters is refused unless asked for, and works inside summon_full_params
    plain = FSDP(nn.Linear(10, 10), compute_device=CPU)
    with pytest.raises((AssertionError, RuntimeError)):
        with plain.summon_full_params():
            plain.reset_parameters()
    resettable = FSDP(nn.Linear(10, 10), allow_reset_parameters=True, compute_device=CPU)
    with resettable.summon_full_params():
        old = resettable.module.weight.detach().clone()
        resettable.reset_parameters()
        assert not torch.equal(old, resettable.module.weight)
    dist.barrier()


def test_single_behaviours():
    spawn_ranks(_single_behaviours, 2, (), backend="gloo")


def _names(rank, world, flatten):
    before = [(n, p.shape) for n, p in _Shared().named_parameters()]
    model = _wrapped(flatten_parameters=flatten)
    _train(model, rank)
    after = list(model.named_parameters())
    if flatten:
        assert "flat_param_0" in after[0][0] and len(after) == 1
    else:
        assert [n for n, _ in after] == [n for n, _ in before]
    with model.summon_full_params():
        inside = list(model.named_parameters())
        assert [n for n, _ in inside] == [n for n, _ in before]           # clean names ...
        assert [p.shape for _, p in inside] == [s for _, s in before]     # ... and full sizes
    assert len(list(model.named_parameters())) == len(after)             # and sharded again afterwards


@pytest.mark.parametrize("flatten", [True, False])
def test_parameter_names_before_and_after_wrapping(flatten):
    spawn_ranks(_names, 2, (flatten,), backend="gloo")


def _clipping(rank, world, norm_type):
    ref = nn.parallel.DistributedDataParallel(_Shared())
    model = _wrapped()
    for m in (ref, model):
        m(_tokens(rank)).float().pow(2).mean().backward()
    want = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.05, norm_type=norm_type)
    got = model.clip_grad_norm_(0.05, norm_type=norm_type)
    torch.testing.assert_close(got.reshape(()), want.reshape(()), atol=1e-6, rtol=1e-5)
    for opt_model in (ref, model):
        torch.optim.SGD(opt_model.parameters(), lr=0.1).step()
    full = model.state_dict()
    for k, v in ref.module.state_dict().items():
        torch.testing.assert_close(full[k], v, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("norm_type", [1, 2, inf])
def test_gradient_clipping_norms(norm_type):
    spawn_ranks(_clipping, 2, (norm_type,), backend="gloo")


def _delayed_step(rank, world):
    """The optimizer step of iteration i runs after the forward of iteration i + 1 has started from the old weights
    (pipelined trainers do this): gradients must survive the intervening forward."""
    ref = nn.parallel.DistributedDataParallel(_Shared())
    model = _wrapped()
    opts = [torch.optim.SGD(m.parameters(), lr=0.1) for m in (ref, model)]
    for m, opt in zip((ref, model), opts):
        opt.zero_grad()
        m(_tokens(rank)).float().pow(2).mean().backward()
        with torch.no_grad():
            m(_tokens(rank + 1))  # a forward in between
        opt.step()
    full = model.state_dict()
    for k, v in ref.module.state_dict().items():
        torch.testing.assert_close(full[k], v, atol=1e-6, rtol=1e-5)
    # evaluation gives the same output with and without no_grad
    model.eval()
    a = model(_tokens(rank))
    with torch.no_grad():
        b = model(_tokens(rank))
    assert torch.equal(a.detach(), b) and not b.requires_grad


def test_delayed_optimizer_step_and_evaluation():
    spawn_ranks(_delayed_step, 2, (), backend="gloo")
