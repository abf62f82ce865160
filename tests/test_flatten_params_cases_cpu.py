"""FlattenParamsWrapper, one case per test function of fairscale tests/nn/misc/test_flatten_params_wrapper.py that needs no
GPU: partial flattening and dtype changes, two groups, nothing to flatten, a module without parameters, parameter counts and
outputs with and without shared weights, the parameter norm after an optimizer step, state-dict equality and loading in
both layouts, and ``unflatten_params`` over tensors supplied from outside.
"""
from collections import OrderedDict

import pytest
import torch
from torch import nn

from fairscale_b200.fair_dev.testing.testing import objects_are_equal
from fairscale_b200.nn.misc import FlattenParamsWrapper


def _transformer(seed=0, groups="all"):
    torch.manual_seed(seed)
    module = nn.Transformer(d_model=32, num_encoder_layers=2, num_decoder_layers=2, dim_feedforward=128, dropout=0.1)
    module.register_buffer("dummy_buffer", torch.tensor(1.0))
    if groups == "all":
        module.param_list, module.flat_param_names = None, None
    else:  # two groups, named
        first = list(module.encoder.layers[1].parameters()) + list(module.decoder.layers[0].parameters())
        second = list(module.encoder.layers[0].parameters()) + list(module.decoder.layers[1].parameters())
        module.param_list, module.flat_param_names = [first, second], ["ordered", "reversed"]
    return module


def _shared_transformer(seed=0):
    module = _transformer(seed)
    for dec, enc in zip(module.decoder.layers, module.encoder.layers):  # decoder layers reuse the encoder's feed-forward
        dec.linear1.weight = enc.linear1.weight
        dec.linear2.weight = enc.linear2.weight
    return module


def _linears(seed=0, groups=None, names=None):
    torch.manual_seed(seed)
    if groups is None:
        module = nn.Sequential(nn.Sequential(nn.Linear(4, 8), nn.Linear(8, 8)), nn.Sequential(nn.Linear(8, 16)), nn.Linear(16, 4))
        module.param_list = None
    else:  # one group per top-level child; together they hold every parameter
        module = nn.Sequential(nn.Sequential(nn.Linear(4, 8), nn.Linear(8, 16)), nn.Linear(16, 4))
        module.param_list = [list(child.parameters()) for child in module]
    module.flat_param_names = names
    return module


BUILDERS = [_linears, _shared_transformer, lambda seed=0: _linears(seed, groups=2),
            lambda seed=0: _linears(seed, groups=2, names=["layer1", "layer2"])]
BUILDER_IDS = ["linears", "shared_transformer", "two_groups", "two_named_groups"]


def _output(module):
    torch.manual_seed(1)
    module.eval()  # no dropout
    if isinstance(getattr(module, "module", module), nn.Transformer):
        src, tgt = torch.rand(20, 8, 32), torch.rand(10, 8, 32)
        return module(src, tgt)
    return module(torch.rand(8, 4))


def _pnorm_after_step(module):
    optim = torch.optim.SGD(module.parameters(), lr=0.01)
    module.train()
    torch.manual_seed(2)
    src, tgt = torch.rand(20, 8, 32), torch.rand(10, 8, 32)
    torch.manual_seed(3)  # dropout masks
    module(src, tgt).sum().backward()
    optim.step()
    return torch.norm(torch.stack([p.detach().norm() for p in module.parameters()]))


def _wrap(module):
    return FlattenParamsWrapper(module, param_list=module.param_list, flat_param_names=module.flat_param_names)


def test_partial_flattening_and_dtype_change():
    module = _transformer()
    total = sum(p.numel() for p in module.parameters())
    chosen = list(module.encoder.layers[1].parameters()) + list(module.decoder.layers[0].parameters())
    chosen_numel = sum(p.numel() for p in chosen)
    module = FlattenParamsWrapper(module, param_list=chosen)
    assert module.flat_param.numel() == chosen_numel
    assert sum(p.numel() for p in module.parameters()) == total
    assert len(list(module.encoder.layers[1].parameters())) == 0 and len(list(module.decoder.layers[0].parameters())) == 0
    assert len(list(module.encoder.layers[0].parameters())) > 0 and len(list(module.decoder.layers[1].parameters())) > 0
    assert module.flat_param.dtype == torch.float32
    module = module.to(dtype=torch.float16)
    assert module.flat_param.dtype == torch.float16
    assert all(p.dtype == torch.float16 for p in module.encoder.layers[0].parameters())


def test_two_groups():
    module = _transformer(groups="two")
    total = sum(p.numel() for p in module.parameters())
    sizes = [sum(p.numel() for p in group) for group in module.param_list]
    module = FlattenParamsWrapper(module, param_list=module.param_list)
    assert [fp.numel() for fp in module.flat_params] == sizes
    assert sum(p.numel() for p in module.parameters()) == total


def test_nothing_to_flatten():
    module = _transformer()
    want_out = _output(module)
    want_state = {k: v.clone() for k, v in module.state_dict().items()}
    module = FlattenParamsWrapper(module, param_list=[[]])
    state = module.state_dict()
    assert state.keys() == want_state.keys()
    for k, v in want_state.items():
        torch.testing.assert_close(state[k], v)
    torch.testing.assert_close(_output(module), want_out)


def test_module_without_parameters():
    class Empty(nn.Module):
        def forward(self, x):
            return x + 1

    x = torch.rand(1)
    module = FlattenParamsWrapper(Empty())
    assert len(list(module.parameters())) == 0 and len(module.state_dict()) == 0
    torch.testing.assert_close(module(x), x + 1)


@pytest.mark.parametrize("build", [_transformer, _shared_transformer], ids=["plain", "shared"])
def test_parameter_count_and_output(build):
    module = build()
    count = sum(p.numel() for p in module.parameters())  # shared weights count once
    want = _output(module)
    flat = FlattenParamsWrapper(module)
    assert sum(p.numel() for p in flat.parameters()) == count == flat.flat_param.numel()
    assert objects_are_equal(_output(flat), want)


def test_shared_weights_parameter_norm_after_a_step():
    want = _pnorm_after_step(_shared_transformer())
    got = _pnorm_after_step(FlattenParamsWrapper(_shared_transformer()))
    torch.testing.assert_close(got, want)


@pytest.mark.parametrize("build", BUILDERS, ids=BUILDER_IDS)
def test_state_dict_is_the_one_of_the_plain_module(build):
    module = build()
    want = OrderedDict((k, v.clone()) for k, v in module.state_dict().items())
    flat = _wrap(module)
    got = flat.state_dict()
    assert got.keys() == want.keys(), f"{list(got.keys())} != {list(want.keys())}"
    assert objects_are_equal(dict(want), dict(got))


@pytest.mark.parametrize("build", BUILDERS, ids=BUILDER_IDS)
def test_plain_state_dict_loads_into_the_wrapper(build):
    module = build()
    state = OrderedDict((k, v.clone()) for k, v in module.state_dict().items())
    want = _output(module)
    flat = _wrap(build(seed=1234))
    assert not objects_are_equal(_output(flat), want)
    flat.load_state_dict(state)  # without the context manager
    assert objects_are_equal(_output(flat), want)
    with flat.unflatten_params():  # and inside it
        flat.load_state_dict(state)
    assert objects_are_equal(_output(flat), want)


@pytest.mark.parametrize("build", BUILDERS, ids=BUILDER_IDS)
def test_flat_state_dict_round_trip(build):
    flat = _wrap(build())
    want = _output(flat)
    state = {k: v.clone() for k, v in flat.flat_state_dict().items()}
    other = _wrap(build(seed=1234))
    other.load_state_dict(state)
    assert objects_are_equal(_output(other), want)


@pytest.mark.parametrize("build", BUILDERS, ids=BUILDER_IDS)
def test_unflatten_params_over_tensors_from_outside(build):
    module = _wrap(build())
    buffers = {k.replace("_fpw_module.", "") for k, _ in module.named_buffers()}

    def snapshot():
        return OrderedDict((k, v.clone()) for k, v in module.state_dict().items())

    kept = [fp.detach().clone() for fp in module.flat_params]
    with module.unflatten_params():
        before = snapshot()
    assert all(not torch.all(fp == 0) for fp in kept)

    outside = [torch.full_like(fp, 42.0) for fp in module.flat_params]
    with module.unflatten_params(flat_params=outside):
        during = snapshot()
    assert during.keys() == before.keys()
    for k, v in during.items():
        torch.testing.assert_close(v, before[k] if k in buffers else torch.full_like(v, 42.0))

    # leaving the context brings the module's own values back
    assert len(module.flat_params) == len(kept)
    for fp, ref in zip(module.flat_params, kept):
        torch.testing.assert_close(fp.detach(), ref)
    with module.unflatten_params():
        assert objects_are_equal(dict(before), dict(snapshot()))

    # loading what was seen inside the context makes the flat parameters equal to the outside tensors
    module.load_state_dict(during)
    for fp, ref in zip(module.flat_params, outside):
        torch.testing.assert_close(fp.detach(), ref)


def test_a_flat_parameter_is_not_flattened_again():
    """An outer wrapper asked to take every parameter of a module that already holds a wrapper refuses; with a parameter list
    that leaves the inner wrapper's flat parameter out, both work side by side."""
    inner = FlattenParamsWrapper(nn.Linear(4, 4))
    with pytest.raises(ValueError, match="Nesting"):
        FlattenParamsWrapper(nn.Sequential(inner, nn.Linear(4, 2)))

    torch.manual_seed(0)
    plain = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 2))
    want_state = {k: v.clone() for k, v in plain.state_dict().items()}
    x = torch.rand(3, 4)
    want = plain(x)
    plain[0] = FlattenParamsWrapper(plain[0])
    outer = FlattenParamsWrapper(plain, param_list=list(plain[1].parameters()))
    torch.testing.assert_close(outer(x), want)
    got_state = outer.state_dict()
    assert got_state.keys() == want_state.keys()
    for k, v in want_state.items():
        torch.testing.assert_close(got_state[k], v)
    assert sorted(p.numel() for p in outer.parameters()) == [4 * 2 + 2, 4 * 4 + 4]
