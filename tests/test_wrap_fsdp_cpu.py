"""auto_wrap with FSDP as the wrapper class (cases of the reference's tests/nn/wrap/test_wrap.py; a stand-in process group, one
process): overriding context defaults at the call, the default size policy on nested sequentials, wrapping the root
without the leftover check, containers that are never wrapped themselves, leaves that are never entered (built in and
user-defined), and a forward / backward through an auto-wrapped model under autocast."""
import functools

import pytest
import torch
import torch.nn.functional as F
from torch import nn

from fairscale_b200.fair_dev.testing.testing import DummyProcessGroup
from fairscale_b200.nn import FullyShardedDataParallel as FSDP
from fairscale_b200.nn import auto_wrap, default_auto_wrap_policy, enable_wrap, wrap

GROUP = DummyProcessGroup(rank=0, size=1)
KW = dict(wrapper_cls=FSDP, process_group=GROUP, compute_device=torch.device("cpu"))


def test_wrap_inside_and_outside_the_context_and_overrides():
    with enable_wrap(flatten_parameters=False, **KW):
        layer = wrap(nn.Linear(5, 5))
        overridden = wrap(nn.Linear(5, 5), flatten_parameters=True)
    assert isinstance(layer, FSDP) and layer.flatten_parameters is False
    assert isinstance(overridden, FSDP) and overridden.flatten_parameters is True
    outside = wrap(nn.Linear(5, 5))
    assert isinstance(outside, nn.Linear)


def test_size_policy_on_nested_sequentials():
    """Leaves of 30 parameters each, threshold 40: a single leaf is too small; the inner pair reaches 60 and is wrapped; the
    root keeps 60 unwrapped parameters of its own and is wrapped too."""
    with enable_wrap(flatten_parameters=False, **KW):
        seq = nn.Sequential(nn.Linear(5, 5), nn.Linear(5, 5), nn.Sequential(nn.Linear(5, 5), nn.Linear(5, 5)))
        model = auto_wrap(seq, auto_wrap_policy=functools.partial(default_auto_wrap_policy, min_num_params=40))
    assert isinstance(model, FSDP)
    assert isinstance(model.module[0], nn.Linear) and isinstance(model.module[1], nn.Linear)
    assert isinstance(model.module[2], FSDP)
    assert isinstance(model.module[2].module[0], nn.Linear) and isinstance(model.module[2].module[1], nn.Linear)


def test_root_wrapped_without_the_leftover_check():
    """Threshold 60: the inner pair is wrapped, which leaves the root with one leaf of 30 parameters - below the threshold, yet
    the root is wrapped when the policy is told to skip that check for it."""
    policy = functools.partial(default_auto_wrap_policy, min_num_params=60, skip_params_check_for_root=True)
    with enable_wrap(flatten_parameters=False, **KW):
        seq = nn.Sequential(nn.Linear(5, 5), nn.Sequential(nn.Linear(5, 5), nn.Linear(5, 5)))
        model = auto_wrap(seq, auto_wrap_policy=policy)
    assert isinstance(model, FSDP) and isinstance(model.module[0], nn.Linear) and isinstance(model.module[1], FSDP)
    # with the check in place the root stays as it is
    with enable_wrap(flatten_parameters=False, **KW):
        seq = nn.Sequential(nn.Linear(5, 5), nn.Sequential(nn.Linear(5, 5), nn.Linear(5, 5)))
        kept = auto_wrap(seq, auto_wrap_policy=functools.partial(default_auto_wrap_policy, min_num_params=60))
    assert isinstance(kept, nn.Sequential) and isinstance(kept[1], FSDP)


def test_containers_are_not_wrapped_but_their_children_may_be():
    policy = functools.partial(default_auto_wrap_policy, min_num_params=40)
    with enable_wrap(flatten_parameters=False, **KW):
        small = auto_wrap(nn.ModuleList([nn.Linear(5, 5), nn.Linear(5, 5)]), auto_wrap_policy=policy)
        large = auto_wrap(nn.ModuleList([nn.Linear(10, 10)]), auto_wrap_policy=policy)
    assert isinstance(small, nn.ModuleList) and isinstance(small[0], nn.Linear) and isinstance(small[1], nn.Linear)  # 60 in total, still not wrapped
    assert isinstance(large, nn.ModuleList) and isinstance(large[0], FSDP)


def test_leaves_that_are_never_entered():
    policy = functools.partial(default_auto_wrap_policy, min_num_params=40)
    with enable_wrap(flatten_parameters=False, **KW):
        model = auto_wrap(nn.Sequential(nn.Linear(10, 10), nn.MultiheadAttention(100, 1)), auto_wrap_policy=policy)
    assert isinstance(model.module[0], FSDP)
    assert isinstance(model.module[1], nn.MultiheadAttention) and isinstance(model.module[1].out_proj, nn.Linear)

    custom = functools.partial(default_auto_wrap_policy, min_num_params=40,
                               force_leaf_modules=default_auto_wrap_policy.FORCE_LEAF_MODULES.union({nn.Linear}))
    with enable_wrap(auto_wrap_policy=custom, flatten_parameters=False, **KW):
        model = auto_wrap(nn.Sequential(nn.Linear(10, 10), nn.ModuleList([nn.Linear(10, 10)])))
    # no inner module could be wrapped, so everything lands in the root's wrapper
    assert isinstance(model, FSDP) and isinstance(model.module[0], nn.Linear) and isinstance(model.module[1], nn.ModuleList)
    assert isinstance(model.module[1][0], nn.Linear)


@pytest.mark.parametrize("mixed_precision", [False, True])
def test_forward_and_backward_through_an_auto_wrapped_model(mixed_precision):
    kw = dict(KW, mixed_precision=mixed_precision)
    if mixed_precision:
        kw["compute_dtype"] = torch.bfloat16
    with enable_wrap(**kw):
        seq = nn.Sequential(nn.Linear(5, 5), nn.Linear(5, 5), nn.Sequential(nn.Linear(5, 5), nn.Linear(5, 5)))
        model = auto_wrap(seq, auto_wrap_policy=functools.partial(default_auto_wrap_policy, min_num_params=40))
    x = torch.rand(1, 5)
    with torch.autocast("cpu", dtype=torch.bfloat16, enabled=mixed_precision):
        out = model(x)
        loss = F.mse_loss(x, out.float())
    loss.backward()
    assert all(p.grad is not None for p in model.parameters())
    assert out.dtype == (torch.bfloat16 if mixed_precision else torch.float32)
