"""enable_wrap / wrap / auto_wrap with a plain wrapper class (no process group needed): kwargs precedence, policies,
excluded containers and forced leaves, nested contexts."""
import functools

import pytest
import torch
from torch import nn

from fairscale_b200.nn import auto_wrap, config_auto_wrap_policy, default_auto_wrap_policy, enable_wrap, wrap


class Box(nn.Module):
    """Stand-in wrapper that records its keyword arguments."""

    def __init__(self, module, **kwargs):
        super().__init__()
        self.module = module
        self.kwargs = kwargs

    def forward(self, *a, **k):
        return self.module(*a, **k)


def test_wrap_is_a_noop_outside_the_context_and_merges_kwargs_inside():
    lin = nn.Linear(2, 2)
    assert wrap(lin, a=1) is lin
    with enable_wrap(wrapper_cls=Box, a=1, b=2):
        tagged = nn.Linear(2, 2)
        tagged.wrapper_config = {"b": 20, "c": 30}
        w = wrap(tagged, c=300)
        plain = wrap(nn.Linear(2, 2))
    assert isinstance(w, Box) and w.kwargs == {"a": 1, "b": 20, "c": 300}  # context < wrapper_config < call overrides
    assert plain.kwargs == {"a": 1, "b": 2}
    assert wrap(lin) is lin  # the context is gone again


def test_nested_contexts_are_refused():
    with enable_wrap(wrapper_cls=Box):
        with pytest.raises(Exception):
            with enable_wrap(wrapper_cls=Box):
                pass


def _count(model, cls=Box):
    return sum(isinstance(m, cls) for m in model.modules())


def test_default_policy_wraps_by_size_and_respects_exclusions():
    model = nn.Sequential(
        nn.Linear(10, 10),                                   # 110 params
        nn.ModuleList([nn.Linear(10, 10), nn.Linear(10, 10)]),  # container is never wrapped itself, children may be
        nn.MultiheadAttention(8, 2),                         # forced leaf: never entered, stays with its parent's wrapper
        nn.Linear(2, 2),                                     # too small
    )
    policy = functools.partial(default_auto_wrap_policy, min_num_params=100)
    with enable_wrap(wrapper_cls=Box, tag="x"):
        out = auto_wrap(model, auto_wrap_policy=policy)
    assert isinstance(out, Box)  # the root holds enough leftover parameters
    inner = out.module
    assert isinstance(inner[0], Box) and inner[0].kwargs == {"tag": "x"}
    assert isinstance(inner[1], nn.ModuleList) and all(isinstance(m, Box) for m in inner[1])
    assert isinstance(inner[2], nn.MultiheadAttention) and not any(isinstance(m, Box) for m in inner[2].modules())
    assert isinstance(inner[3], nn.Linear)
    # a large threshold wraps nothing
    with enable_wrap(wrapper_cls=Box):
        untouched = auto_wrap(nn.Sequential(nn.Linear(3, 3), nn.Linear(3, 3)), auto_wrap_policy=functools.partial(default_auto_wrap_policy, min_num_params=10**6))
    assert _count(untouched) == 0


def test_config_policy_wraps_exactly_the_tagged_modules():
    a, b, c = nn.Linear(4, 4), nn.Linear(4, 4), nn.Linear(4, 4)
    b.wrapper_config = {"flag": True}
    deep = nn.Sequential(c)
    c.wrapper_config = {}
    model = nn.Sequential(a, b, deep)
    with enable_wrap(config_auto_wrap_policy, wrapper_cls=Box):
        out = auto_wrap(model)
    assert isinstance(out[1], Box) and out[1].kwargs == {"flag": True}
    assert isinstance(out[2][0], Box) and isinstance(out[0], nn.Linear) and not isinstance(out, Box)
    x = torch.randn(2, 4)
    assert out(x).shape == (2, 4)
