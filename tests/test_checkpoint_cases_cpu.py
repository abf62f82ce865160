"""checkpoint_wrapper, case by case on CPU (cases of the reference's tests/nn/checkpoint/test_checkpoint_activations.py and
test_checkpoint_activations_norm.py): several inputs and outputs under every combination of wrapped branches, list inputs,
switching checkpointing off, how often a block runs depending on who needs gradients (also through FlattenParamsWrapper
and with non-tensor arguments), normalisation layers, and both import paths."""
import pytest
import torch
from torch import nn
from torch.optim import SGD

from fairscale_b200.fair_dev.testing.testing import objects_are_equal
from fairscale_b200.nn import checkpoint_wrapper
from fairscale_b200.nn.checkpoint.checkpoint_activations import disable_checkpointing
from fairscale_b200.nn.misc import FlattenParamsWrapper


def _loss_and_gnorm(model, *inputs, **kw):
    out = model(*inputs, **kw)
    if isinstance(out, tuple):
        out = torch.cat(out)
    loss = out.sum()
    loss.backward()
    gnorm = torch.norm(torch.stack([torch.norm(p.grad.detach()) for p in model.parameters()]))
    return {"loss": loss.item(), "gnorm": gnorm.item()}


class _Basic(nn.Module):
    def __init__(self, checkpointed=False, offload=False):
        super().__init__()
        torch.manual_seed(0)
        self.ffn = nn.Sequential(nn.Linear(32, 128), nn.Dropout(p=0.5), nn.Linear(128, 32))
        if checkpointed:
            self.ffn = checkpoint_wrapper(self.ffn, offload)
        self.out = nn.Linear(32, 1)

    def forward(self, x):
        return self.out(self.ffn(x))


def test_loss_and_gradient_norm_with_dropout_inside():
    x = torch.rand(2, 16, 32).requires_grad_(True)
    results = []
    for kw in (dict(), dict(checkpointed=True), dict(checkpointed=True, offload=True)):
        torch.manual_seed(1)  # the same dropout mask for every variant
        results.append(_loss_and_gnorm(_Basic(**kw), x))
    assert results[0] == results[1] == results[2], results


class _TwoBranches(nn.Module):
    def __init__(self, multiout, config):
        super().__init__()
        torch.manual_seed(0)
        self.multiout = multiout
        self.conv1 = nn.Sequential(nn.Conv2d(1, 5, 3), nn.ReLU(), nn.Conv2d(5, 5, 3))
        self.conv2 = nn.Sequential(nn.Conv2d(3, 5, 3), nn.ReLU(), nn.Conv2d(5, 5, 3))
        if config & 1:
            self.conv1 = checkpoint_wrapper(self.conv1)
        if config & 2:
            self.conv2 = checkpoint_wrapper(self.conv2)

    def forward(self, x1, x2=None):
        a, b = self.conv1(x1), self.conv2(x2)
        return (a, b) if self.multiout else a + b


@pytest.mark.parametrize("multiout", [True, False])
@pytest.mark.parametrize("config", [1, 2, 3])
def test_two_inputs_and_two_outputs(multiout, config):
    in1 = torch.rand(4, 1, 16, 16).requires_grad_(True)
    in2 = torch.rand(4, 3, 16, 16).requires_grad_(True)
    plain = _loss_and_gnorm(_TwoBranches(multiout, 0), in1, x2=in2)
    wrapped = _loss_and_gnorm(_TwoBranches(multiout, config), in1, x2=in2)
    assert plain == wrapped, (plain, wrapped)


class _Counting(nn.Module):
    def __init__(self):
        super().__init__()
        self.cnt = 0
        self.linear = nn.Linear(2, 2)

    def forward(self, x):
        self.cnt += 1
        return [self.linear(i) for i in x] if isinstance(x, (list, tuple)) else self.linear(x)


def test_list_input_and_switching_checkpointing_off():
    first, second = checkpoint_wrapper(_Counting()), _Counting()
    model = nn.Sequential(first, second)
    out = model([torch.rand(4, 2), torch.rand(4, 2)])
    assert first.cnt == 1 and second.cnt == 1
    sum(o.sum() for o in out).backward()
    assert first.cnt == 2 and second.cnt == 1  # the wrapped block ran again in backward

    x = torch.rand(4, 2)
    on, off = checkpoint_wrapper(_Counting()), checkpoint_wrapper(_Counting())
    on(x).sum().backward()
    assert on.cnt == 2
    with disable_checkpointing():
        off(x).sum().backward()
    assert off.cnt == 1
    off(x).sum().backward()  # and it is on again outside the context
    assert off.cnt == 3


def _chain(wrap=lambda m: m):
    return nn.Sequential(*[wrap(checkpoint_wrapper(_Counting())) for _ in range(4)])


@pytest.mark.parametrize("flat", [False, True])
def test_blocks_run_again_only_when_something_upstream_needs_gradients(flat):
    wrap = FlattenParamsWrapper if flat else (lambda m: m)
    x = torch.rand(4, 2)
    model = _chain(wrap)
    for i in range(3):
        model[i].requires_grad_(False)
    model(x).sum().backward()
    assert [m.cnt for m in model] == [1, 1, 1, 2]  # only the last block has anything to compute in backward

    model = _chain(wrap)
    model[1].requires_grad_(False)
    model[2].requires_grad_(False)
    model(x).sum().backward()
    assert [m.cnt for m in model] == [2, 2, 2, 2]  # the first block needs gradients, so they flow through all of them


class _Mixed(nn.Module):
    def __init__(self):
        super().__init__()
        self.cnt = 0
        self.linear = nn.Linear(2, 2)

    def forward(self, x, y, z):
        self.cnt += 1
        return self.linear(x + y), z + [self.cnt], ["hi"]


@pytest.mark.parametrize("freeze_first", [True, False])
def test_non_tensor_arguments_between_blocks(freeze_first):
    x = torch.rand(4, 2)
    m1, m2, m3, m4 = checkpoint_wrapper(_Counting()), checkpoint_wrapper(_Counting()), checkpoint_wrapper(_Mixed()), checkpoint_wrapper(_Counting())
    if freeze_first:
        m1.requires_grad_(False)
    m2.requires_grad_(False)
    out, trail, words = m3(m1(x), m2(x), ["bye"])
    assert trail == ["bye", 1] and words == ["hi"]
    m4(out).sum().backward()
    assert (m1.cnt, m2.cnt, m3.cnt, m4.cnt) == ((1, 1, 2, 2) if freeze_first else (2, 1, 2, 2))


@pytest.mark.parametrize("norm", [nn.LayerNorm, nn.BatchNorm2d])
def test_normalisation_layers_train_to_the_same_state(norm):
    def make(checkpointed):
        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(3, 2), norm(2))
        return checkpoint_wrapper(model) if checkpointed else model

    x = torch.rand(2, 2, 3, 3, requires_grad=True)
    plain, wrapped = make(False), make(True)
    wrapped.load_state_dict(plain.state_dict())
    assert objects_are_equal(plain.state_dict(), wrapped.state_dict())
    for model in (plain, wrapped):
        opt = SGD(model.parameters(), lr=0.1)
        model(x).sum().backward()
        opt.step()
    assert objects_are_equal(plain.state_dict(), wrapped.state_dict())  # running statistics counted once, same update
    # half precision layers refuse to run on a CPU with or without the wrapper
    half = checkpoint_wrapper(nn.Sequential(nn.Linear(3, 2), norm(2)).half())
    try:
        half(x.detach().half().requires_grad_()).sum().backward()
    except RuntimeError:
        pass


def test_both_import_paths_give_the_same_function():
    from fairscale_b200.nn.checkpoint import checkpoint_wrapper as new_path
    from fairscale_b200.nn.misc import checkpoint_wrapper as old_path

    ffn = nn.Sequential(nn.Linear(32, 128), nn.Dropout(p=0.5), nn.Linear(128, 32))
    assert new_path is checkpoint_wrapper
    wrapped = old_path(ffn, {})
    assert wrapped(torch.rand(2, 32)).shape == (2, 32)
