"""Building blocks on one CPU process: FlattenParamsWrapper (shared weights, several flat groups, pickling, training parity,
empty modules), Param / GradBucket life cycle and error messages, and checkpoint_wrapper (keyword and non-tensor
arguments, non-tensor outputs, dropout replay, batch-norm statistics counted once, nesting, mixed precision autocast).
Cases of the reference's tests/nn/misc/test_flatten_params_wrapper.py, test_param_bucket.py, test_grad_bucket.py and
tests/nn/checkpoint/test_checkpoint_activations*.py."""
import copy
import pickle

import pytest
import torch
from torch import nn

from fairscale_b200.nn import checkpoint_wrapper
from fairscale_b200.nn.checkpoint.checkpoint_activations import disable_checkpointing, is_checkpointing, is_recomputing
from fairscale_b200.nn.misc import FlattenParamsWrapper
from fairscale_b200.nn.misc.param_bucket import GradBucket, ParamBucket


# ------------------------------------------------------------------------------------------------ FlattenParamsWrapper
class _Tied(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.embed = nn.Embedding(11, 6)
        self.body = nn.Sequential(nn.Linear(6, 6), nn.Tanh())
        self.out = nn.Linear(6, 11, bias=False)
        self.out.weight = self.embed.weight  # shared

    def forward(self, tokens):
        return self.out(self.body(self.embed(tokens)))


def _train(model, steps=3):
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        tokens = torch.randint(0, 11, (4, 5), generator=g)
        opt.zero_grad()
        nn.functional.cross_entropy(model(tokens).flatten(0, 1), tokens.flatten()).backward()
        opt.step()
    return model


def test_flat_wrapper_trains_like_the_plain_module_with_a_shared_weight():
    plain = _train(_Tied())
    flat = _train(FlattenParamsWrapper(_Tied()))
    assert len(list(flat.parameters())) == 1  # the shared weight is stored once
    assert flat.flat_param.numel() == sum(p.numel() for p in plain.parameters())
    for (k, v), (k2, w) in zip(plain.state_dict().items(), flat.state_dict().items()):
        assert k == k2  # the unflattened state dict has the original names, shared entries included
        torch.testing.assert_close(w, v, atol=1e-6, rtol=1e-5)
    # and the flat one has a single tensor
    assert list(flat.flat_state_dict().keys()) == ["flat_param_0"]


def test_flat_wrapper_groups_pickle_and_state_dict_round_trips():
    torch.manual_seed(2)
    net = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4), nn.Linear(4, 2))
    groups = [list(net[0].parameters()), list(net[2].parameters())]  # the middle layer stays unflattened
    wrapped = FlattenParamsWrapper(net, param_list=groups, flat_param_names=["first", "last"])
    names = [n for n, _ in wrapped.named_parameters()]
    assert sorted(names) == sorted(["flat_param_first", "flat_param_last", "_fpw_module.1.weight", "_fpw_module.1.bias"])
    x = torch.randn(3, 4)
    y = wrapped(x)

    clone = pickle.loads(pickle.dumps(wrapped))
    torch.testing.assert_close(clone(x), y)

    # flat <-> unflat state dicts load into each other's module
    other = FlattenParamsWrapper(copy.deepcopy(nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4), nn.Linear(4, 2))), param_list=None)
    plain_sd = wrapped.state_dict()
    assert all(not k.startswith("flat_param") for k in plain_sd)
    other.load_state_dict(plain_sd)
    torch.testing.assert_close(other(x), y)
    wrapped.load_state_dict(wrapped.flat_state_dict())
    torch.testing.assert_close(wrapped(x), y)

    # a parameter may not sit in two groups
    with pytest.raises((AssertionError, ValueError)):
        FlattenParamsWrapper(nn.Linear(2, 2), param_list=[[p for p in nn.Linear(2, 2).parameters()]] * 2)


def test_flat_wrapper_without_parameters_and_unflatten_context():
    empty = FlattenParamsWrapper(nn.Sequential(nn.ReLU(), nn.Tanh()))
    assert list(empty.parameters()) == [] and torch.equal(empty(torch.ones(2)), torch.tanh(torch.ones(2)))

    wrapped = FlattenParamsWrapper(nn.Linear(3, 2))
    with wrapped.unflatten_params():
        assert isinstance(wrapped.module.weight, nn.Parameter) and not hasattr(wrapped, "flat_param_0")
        wrapped.module.weight.data.fill_(0.5)
    assert wrapped.is_flattened and float(wrapped.flat_param[0]) == 0.5  # edits made inside the context persist
    # an external flat tensor can stand in for the data
    with wrapped.unflatten_params(flat_params=[torch.zeros_like(wrapped.flat_param)]):
        assert float(wrapped.module.weight.abs().sum()) == 0.0
    assert float(wrapped.flat_param[0]) == 0.5


# ------------------------------------------------------------------------------------------------ buckets
def test_param_bucket_life_cycle_and_errors():
    a, b = torch.arange(6.0).view(2, 3), torch.ones(4)
    bucket = ParamBucket(size=ParamBucket.required_size([a, b], align=4), dtype=torch.float32, device=torch.device("cpu"), align=4)
    bucket.add_param(a)
    bucket.add_param(b)
    assert a.data_ptr() == bucket.buffer.data_ptr() and b.data_ptr() == bucket.buffer.data_ptr() + 8 * 4  # second window aligned to 4 elements
    assert torch.equal(a, torch.arange(6.0).view(2, 3)) and torch.equal(b, torch.ones(4))
    bucket.buffer.mul_(2)
    assert float(a[1, 2]) == 10.0  # the members are views
    with pytest.raises(AssertionError):
        bucket.add_param(a)  # twice
    with pytest.raises(AssertionError):
        bucket.add_param(torch.ones(2, dtype=torch.float16))  # wrong dtype
    with pytest.raises(AssertionError):
        bucket.add_param(torch.ones(64))  # does not fit
    bucket.to(torch.device("cpu"), dtype=torch.float64)
    assert a.dtype == torch.float64 and a.data_ptr() == bucket.buffer.data_ptr()


def test_grad_bucket_check_in_collapse_rebuild_and_shrink():
    ps = [nn.Parameter(torch.randn(3, 3)), nn.Parameter(torch.randn(5))]
    ps[0].grad = torch.full((3, 3), 2.0)
    bucket = GradBucket(64, dtype=torch.float32, device=torch.device("cpu"), destination=1)
    for p in ps:
        assert bucket.can_add_grad_view(p)
        bucket.add_grad(p)
    assert bucket.destination == 1 and not bucket.can_add_grad_view(ps[0])
    assert float(ps[0].grad.sum()) == 18.0 and float(ps[1].grad.abs().sum()) == 0.0  # existing value kept, missing one is zero
    bucket.shrink()
    assert bucket.buffer.numel() == 14 and ps[1].grad.data_ptr() == bucket.buffer.data_ptr() + 9 * 4

    bucket.reset_checked_in()
    assert not bucket.all_checked_in
    bucket.params_checked_in = 2
    assert bucket.all_checked_in

    bucket.collapse()
    assert ps[0].grad is None and bucket.buffer.numel() == 0
    bucket.rebuild()
    assert ps[0].grad is not None and float(ps[0].grad.abs().sum()) == 0.0 and bucket.buffer.numel() == 14
    bucket.zero()
    # a gradient that was replaced comes back into its window
    ps[1].grad = torch.ones(5)
    bucket.readopt_grad(ps[1])
    assert ps[1].grad.data_ptr() == bucket.buffer.data_ptr() + 9 * 4 and float(bucket.buffer[9:].sum()) == 5.0


# ------------------------------------------------------------------------------------------------ checkpoint_wrapper
class _Odd(nn.Module):
    """Keyword tensors, a non-tensor flag in, and a (tensor, string, tensor) tuple out."""

    def __init__(self):
        super().__init__()
        torch.manual_seed(4)
        self.lin = nn.Linear(4, 4)
        self.calls = 0

    def forward(self, x, scale=None, flip=False, note="-"):
        self.calls += 1
        y = self.lin(x)
        if scale is not None:
            y = y * scale
        return (-y if flip else y), note.upper(), y.sum(dim=-1)


def test_checkpoint_keyword_arguments_and_non_tensor_values():
    plain, ck = _Odd(), checkpoint_wrapper(_Odd())
    x = torch.randn(3, 4, requires_grad=True)
    x2 = x.detach().clone().requires_grad_()
    s = torch.full((4,), 1.5, requires_grad=True)
    s2 = s.detach().clone().requires_grad_()
    a = plain(x, scale=s, flip=True, note="abc")
    b = ck(x2, scale=s2, flip=True, note="abc")
    assert b[1] == "ABC" and isinstance(b, tuple) and len(b) == 3
    (a[0].sum() + a[2].sum()).backward()
    (b[0].sum() + b[2].sum()).backward()
    torch.testing.assert_close(x2.grad, x.grad)
    torch.testing.assert_close(s2.grad, s.grad)
    for p, q in zip(plain.parameters(), ck.parameters()):
        torch.testing.assert_close(q.grad, p.grad)
    assert ck.calls == 2  # forward without grad, then the replay


def test_checkpoint_replays_dropout_and_counts_batch_norm_once():
    torch.manual_seed(0)
    drop = checkpoint_wrapper(nn.Sequential(nn.Linear(8, 8), nn.Dropout(0.5), nn.Linear(8, 8)))
    x = torch.randn(16, 8, requires_grad=True)
    torch.manual_seed(123)
    out = drop(x)
    torch.manual_seed(999)  # whatever happened to the generator in between, the replay uses the forward's masks
    out.sum().backward()
    g1 = x.grad.clone()
    plain = copy.deepcopy(drop)
    x.grad = None
    with disable_checkpointing():
        torch.manual_seed(123)
        plain(x).sum().backward()
    torch.testing.assert_close(x.grad, g1)

    bn = checkpoint_wrapper(nn.Sequential(nn.Linear(4, 4), nn.BatchNorm1d(4)))
    ref = copy.deepcopy(bn)
    y = torch.randn(6, 4, requires_grad=True)
    bn(y).sum().backward()
    with disable_checkpointing():
        ref(y).sum().backward()
    # running statistics were updated by the first forward only, not again by the replay
    torch.testing.assert_close(bn[1].running_mean, ref[1].running_mean)
    torch.testing.assert_close(bn[1].running_var, ref[1].running_var)
    assert int(bn[1].num_batches_tracked) == 1


def test_checkpoint_nesting_flags_and_autocast():
    seen = []

    class Probe(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(4, 4)

        def forward(self, x):
            seen.append((is_checkpointing(), is_recomputing(), torch.is_autocast_enabled("cpu")))
            return self.lin(x)

    inner = checkpoint_wrapper(Probe())
    outer = checkpoint_wrapper(nn.Sequential(nn.Linear(4, 4), inner))
    x = torch.randn(2, 4, requires_grad=True)
    with torch.autocast("cpu", dtype=torch.bfloat16):
        out = outer(x)
    out.float().sum().backward()
    # first pass: inside the outer checkpoint's no-grad forward; replay of the outer runs the inner's own first pass and replay
    assert seen[0][0] and not seen[0][1]
    assert any(rec for _, rec, _ in seen[1:])
    assert all(autocast for _, _, autocast in seen), "the replay runs under the autocast state of the forward"
    assert x.grad is not None and all(p.grad is not None for p in outer.parameters())
