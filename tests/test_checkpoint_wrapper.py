import gc
import weakref

import pytest
import torch
from torch import nn

from fairscale_b200.nn.checkpoint import checkpoint_wrapper, disable_checkpointing, is_checkpointing, is_recomputing
from fairscale_b200.nn.misc import FlattenParamsWrapper


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(8, 16)
        self.drop = nn.Dropout(0.3)
        self.l2 = nn.Linear(16, 8)
        self.bn = nn.BatchNorm1d(8)
        self.calls = []

    def forward(self, x, scale=1.0, tag=None):
        self.calls.append((is_checkpointing(), is_recomputing()))
        y = self.bn(self.l2(self.drop(torch.relu(self.l1(x))))) * scale
        return (y, tag) if tag is not None else y


@pytest.mark.parametrize("offload", [False, True])
def test_matches_plain_module(offload):
    torch.manual_seed(0)
    plain, ckpt = Block(), Block()
    ckpt.load_state_dict(plain.state_dict())
    checkpoint_wrapper(ckpt, offload_to_cpu=offload)
    x1 = torch.randn(4, 8, requires_grad=True)
    x2 = x1.detach().clone().requires_grad_()
    torch.manual_seed(5)
    y1 = plain(x1, scale=2.0)
    torch.manual_seed(5)
    y2, tag = ckpt(x2, scale=2.0, tag="hello")
    assert tag == "hello"
    torch.testing.assert_close(y1, y2)
    y1.sum().backward()
    y2.sum().backward()
    torch.testing.assert_close(x1.grad, x2.grad)
    for a, b in zip(plain.parameters(), ckpt.parameters()):
        torch.testing.assert_close(a.grad, b.grad)
    # BatchNorm statistics are updated exactly once
    torch.testing.assert_close(plain.bn.running_mean, ckpt.bn.running_mean)
    assert ckpt.bn.num_batches_tracked.item() == 1
    assert ckpt.calls == [(True, False), (False, True)]


def test_noop_paths_and_errors():
    m = checkpoint_wrapper(Block())
    with torch.no_grad():
        m(torch.randn(2, 8))
    assert m.calls == [(False, False)]
    with disable_checkpointing():
        m(torch.randn(2, 8, requires_grad=True)).sum().backward()
    assert m.calls[-1] == (False, False)
    frozen = checkpoint_wrapper(nn.Linear(3, 3))
    for p in frozen.parameters():
        p.requires_grad = False
    out = frozen(torch.randn(2, 3))
    assert not out.requires_grad


def test_flattened_module_outputs_require_grad():
    inner = checkpoint_wrapper(nn.Linear(4, 4))
    fpw = FlattenParamsWrapper(inner)
    out = fpw(torch.randn(2, 4))
    assert out.requires_grad
    out.sum().backward()
    assert fpw.flat_param.grad is not None


def test_no_reference_cycle():
    m = checkpoint_wrapper(nn.Linear(2, 2))
    ref = weakref.ref(m)
    del m
    gc.collect()
    assert ref() is None
