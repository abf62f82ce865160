"""FSDP state dicts over the configuration grid of the reference's tests/nn/data_parallel/test_fsdp_state_dict.py (gloo ranks,
bf16 as the low-precision type): local state dicts saved, loaded and changed by training; asking twice; before any forward;
a trained state loaded into a fresh wrapper; nested wrappers against DistributedDataParallel; dtypes of what comes back
(fp32 master values under mixed precision, the parameters' own type for a model cast as a whole); and a subclass whose
``state_dict`` is its ``local_state_dict`` without recursing for ever."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import objects_are_equal, spawn_ranks
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP

CPU = torch.device("cpu")
CONFIGS = [dict(flatten_parameters=f, mixed_precision=m) for f in (True, False) for m in (True, False)]


def _config(config):
    out = dict(config, compute_device=CPU)
    if out.get("mixed_precision"):
        out["compute_dtype"] = torch.bfloat16
    return out


class _SharedParams(nn.Module):
    """Embedding tied to the output projection, a bias kept as a bare parameter, a buffer."""

    def __init__(self, d_vocab=23, d_model=16):
        super().__init__()
        torch.manual_seed(0)
        self.embed_tokens = nn.Embedding(d_vocab, d_model)
        self.body = nn.Sequential(nn.Linear(d_model, d_model), nn.Tanh(), nn.Linear(d_model, d_model))
        self.output_proj = nn.Linear(d_model, d_vocab, bias=False)
        self.output_proj.weight = self.embed_tokens.weight
        self.vocab_bias = nn.Parameter(torch.zeros(d_vocab))
        self.register_buffer("long_buffer", torch.zeros(1, dtype=torch.long))

    def forward(self, tokens):
        self.long_buffer += 1
        return self.output_proj(self.body(self.embed_tokens(tokens))) + self.vocab_bias


class _Nested(nn.Module):
    def __init__(self, wrap):
        super().__init__()
        torch.manual_seed(0)
        self.module = nn.Sequential(nn.Linear(8, 4), wrap(nn.Sequential(wrap(nn.Linear(4, 16)), nn.Linear(16, 16))), wrap(nn.Linear(16, 4)),
                                    nn.Linear(4, 8))

    def forward(self, x):
        return self.module(x)


def _train(model, rank, steps, tokens=True):
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    g = torch.Generator().manual_seed(10 + rank)
    for _ in range(steps):
        x = torch.randint(0, 23, (4, 6), generator=g) if tokens else torch.randn(4, 8, generator=g)
        opt.zero_grad()
        model(x).float().pow(2).mean().backward()
        opt.step()


def _local_state(rank, world, config):
    model = FSDP(_SharedParams(), **_config(config))
    first = model.local_state_dict()
    before = {k: v.clone() for k, v in first.items()}
    assert len(first) > 0
    model.load_local_state_dict(first)
    key = "flat_param_0" if config["flatten_parameters"] else "embed_tokens.weight"
    assert first[key].dtype == torch.float32  # the master values, whatever the compute type
    if not config["flatten_parameters"]:
        torch.testing.assert_close(first[key], model.module.state_dict()[key])
    _train(model, rank, 6)
    second = model.local_state_dict()
    model.load_local_state_dict(second)
    assert first.keys() == second.keys()
    buffers = {"long_buffer"}
    unchanged = [k for k in before if k not in buffers and torch.equal(before[k], second[k])]
    assert not unchanged, f"not changed by training: {unchanged}"
    assert int(second["long_buffer"]) == 6


@pytest.mark.parametrize("config", [CONFIGS[0], CONFIGS[3]], ids=["flat_mixed", "unflat_full"])
def test_local_state_dict_is_saved_loaded_and_trained(config):
    spawn_ranks(_local_state, 2, (config,), backend="gloo")


def _asking(rank, world, config):
    model = FSDP(_SharedParams(), **_config(config))
    early = model.state_dict()  # before any forward
    for name in ("embed_tokens.weight", "vocab_bias"):
        assert early[name].dtype == torch.float32
    plain = _SharedParams().state_dict()
    assert set(early) == set(plain) and all(torch.equal(early[k], plain[k]) for k in plain)
    _train(model, rank, 1)
    a, b = model.state_dict(), model.state_dict()  # twice in a row
    assert objects_are_equal(a, b) and not torch.equal(a["vocab_bias"], early["vocab_bias"])
    _train(model, rank, 1)  # and training goes on afterwards


@pytest.mark.parametrize("config", CONFIGS, ids=lambda c: f"flat{int(c['flatten_parameters'])}_mixed{int(c['mixed_precision'])}")
def test_state_dict_before_forward_and_twice(config):
    spawn_ranks(_asking, 2, (config,), backend="gloo")


def _into_a_fresh_wrapper(rank, world, config):
    model = FSDP(_SharedParams(), **_config(config))
    _train(model, rank, 2)
    trained = model.state_dict()
    plain = _SharedParams()
    plain.load_state_dict(trained)  # the keys and shapes of the bare model
    fresh = FSDP(plain, **_config(config))
    assert objects_are_equal(fresh.state_dict(), trained)
    _train(fresh, rank, 2)
    assert not torch.equal(fresh.state_dict()["vocab_bias"], trained["vocab_bias"])
    # a state dict with a missing key is refused
    broken = dict(trained)
    broken.pop("vocab_bias")
    with pytest.raises((RuntimeError, KeyError)):
        model.load_state_dict(broken)
    dist.barrier()


@pytest.mark.parametrize("config", CONFIGS, ids=lambda c: f"flat{int(c['flatten_parameters'])}_mixed{int(c['mixed_precision'])}")
def test_trained_state_loads_into_a_fresh_wrapper(config):
    spawn_ranks(_into_a_fresh_wrapper, 2, (config,), backend="gloo")


def _nested(rank, world, config):
    ddp = nn.parallel.DistributedDataParallel(_Nested(lambda m: m))
    _train(ddp, rank, 2, tokens=False)
    want = {k: v.clone() for k, v in ddp.module.state_dict().items()}
    cfg = _config(dict(config, mixed_precision=False))  # compared with fp32 DDP
    model = FSDP(_Nested(lambda m: FSDP(m, **cfg)), **cfg)
    _train(model, rank, 2, tokens=False)
    got = {k: v.clone() for k, v in model.state_dict().items()}
    model.load_state_dict(got)
    again = model.state_dict()
    assert want.keys() == again.keys()
    for k in want:
        torch.testing.assert_close(again[k], want[k], atol=1e-6, rtol=1e-5)
    local = {k: v.clone() for k, v in model.local_state_dict().items()}
    model.load_local_state_dict(local)
    reloaded = model.local_state_dict()
    assert reloaded.keys() == local.keys() and all(torch.equal(reloaded[k], local[k]) for k in local)


@pytest.mark.parametrize("flatten", [True, False])
def test_nested_wrappers_against_ddp(flatten):
    spawn_ranks(_nested, 2, (dict(flatten_parameters=flatten),), backend="gloo")


def _dtypes(rank, world, mixed, whole_model_cast):
    model = _SharedParams()
    cfg = dict(compute_device=CPU, mixed_precision=mixed)
    if whole_model_cast:
        model = model.bfloat16()
        cfg["compute_dtype"] = torch.bfloat16
    elif mixed:
        cfg["compute_dtype"] = torch.bfloat16
    fsdp = FSDP(model, **cfg)
    _train(fsdp, rank, 1)
    want = torch.bfloat16 if whole_model_cast else torch.float32
    for k, v in fsdp.state_dict().items():
        assert v.device.type == "cpu"
        if v.is_floating_point():
            assert v.dtype == want, (k, v.dtype)
    kept = FSDP(copy.deepcopy(_SharedParams()), state_dict_device=CPU, **cfg) if not whole_model_cast else None
    if kept is not None:
        assert all(v.device.type == "cpu" for v in kept.state_dict().values())


@pytest.mark.parametrize("mixed,whole_model_cast", [(False, False), (True, False), (False, True)])
def test_dtypes_of_the_returned_tensors(mixed, whole_model_cast):
    spawn_ranks(_dtypes, 2, (mixed, whole_model_cast), backend="gloo")


def _subclass(rank, world):
    class LocalOnly(FSDP):
        def __init__(self):
            super().__init__(module=nn.Linear(100, 100), compute_device=CPU)

        def state_dict(self, *args, **kwargs):
            return self.local_state_dict(*args, **kwargs)

    m = LocalOnly()
    sd = m.state_dict()
    assert set(sd) == {"flat_param_0"} and sd["flat_param_0"].numel() == (100 * 100 + 100 + world - 1) // world


def test_subclass_whose_state_dict_is_the_local_one():
    spawn_ranks(_subclass, 2, (), backend="gloo")
