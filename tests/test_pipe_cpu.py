"""Pipe on CPU devices: parity with the un-piped model, checkpoint modes, skip connections, errors, balance."""
import pytest
import torch
from torch import nn

from fairscale_b200.nn.pipe import Pipe, is_checkpointing, is_recomputing
from fairscale_b200.nn.pipe.balance import balance_cost, blockpartition
from fairscale_b200.nn.pipe.batchnorm import DeferredBatchNorm
from fairscale_b200.nn.pipe.pipeline import clock_cycles
from fairscale_b200.nn.pipe.skip import Namespace, pop, skippable, stash, verify_skippables


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 4))


@pytest.mark.parametrize("checkpoint", ["always", "except_last", "never"])
@pytest.mark.parametrize("chunks", [1, 3, 4])
def test_parity_with_sequential(checkpoint, chunks):
    ref = _model()
    piped = Pipe(_model(), balance=[2, 2, 1], devices=["cpu"] * 3, chunks=chunks, checkpoint=checkpoint)
    x = torch.randn(6, 8)
    y_ref = ref(x)
    y = piped(x)
    torch.testing.assert_close(y, y_ref)
    y_ref.pow(2).sum().backward()
    y.pow(2).sum().backward()
    for a, b in zip(ref.parameters(), piped.parameters()):
        torch.testing.assert_close(a.grad, b.grad)


def test_clock_cycles():
    assert list(clock_cycles(3, 3)) == [[(0, 0)], [(1, 0), (0, 1)], [(2, 0), (1, 1), (0, 2)], [(2, 1), (1, 2)], [(2, 2)]]


def test_errors_and_container_protocol():
    with pytest.raises(TypeError):
        Pipe(nn.Linear(2, 2), balance=[1])
    with pytest.raises(ValueError):
        Pipe(_model(), balance=None)
    with pytest.raises(ValueError):
        Pipe(_model(), balance=[2, 2], devices=["cpu"] * 2)
    with pytest.raises(ValueError):
        Pipe(_model(), balance=[5, 0], devices=["cpu"] * 2)
    with pytest.raises(IndexError):
        Pipe(_model(), balance=[2, 2, 1], devices=["cpu"])
    with pytest.raises(ValueError):
        Pipe(_model(), balance=[5], devices=["cpu"], chunks=0)
    with pytest.raises(ValueError):
        Pipe(_model(), balance=[5], devices=["cpu"], checkpoint="sometimes")
    lin = nn.Linear(2, 2)
    with pytest.raises(ValueError):
        Pipe(nn.Sequential(lin, lin), balance=[2], devices=["cpu"])
    p = Pipe(_model(), balance=[3, 2], devices=["cpu"] * 2)
    assert len(p) == 5 and isinstance(p[0], nn.Linear) and isinstance(p[-1], nn.Linear)
    assert len(list(p)) == 5
    with pytest.raises(TypeError):
        p.cuda()
    with pytest.raises(TypeError):
        p.to("cpu")
    with pytest.raises(TypeError):
        p("not a tensor")
    out = p(torch.randn(2, 8))  # batch smaller than chunks is fine
    assert out.shape == (2, 4)


def test_exception_propagates_from_worker():
    class Boom(nn.Module):
        def forward(self, x):
            raise RuntimeError("boom")

    p = Pipe(nn.Sequential(nn.Linear(2, 2), Boom()), balance=[1, 1], devices=["cpu"] * 2, chunks=2)
    with pytest.raises(RuntimeError, match="boom"):
        p(torch.randn(4, 2))


def test_recompute_flags_and_deferred_batchnorm():
    seen = []

    class Probe(nn.Module):
        def forward(self, x):
            seen.append((is_checkpointing(), is_recomputing()))
            return x * 2

    p = Pipe(nn.Sequential(nn.Linear(2, 2), Probe()), balance=[1, 1], devices=["cpu"] * 2, chunks=2, checkpoint="always")
    p(torch.randn(4, 2, requires_grad=True)).sum().backward()
    assert (True, False) in seen and (False, True) in seen

    torch.manual_seed(0)
    bn = nn.BatchNorm2d(3)
    dbn = DeferredBatchNorm.convert_deferred_batch_norm(nn.Sequential(nn.BatchNorm2d(3)), chunks=2)[0]
    x = torch.randn(4, 3, 5, 5)
    bn(x)
    for chunk in x.chunk(2):
        dbn(chunk)
    torch.testing.assert_close(dbn.running_mean, bn.running_mean, atol=1e-6, rtol=1e-5)
    assert dbn.num_batches_tracked.item() == 1


def test_skip_connections_across_partitions():
    @skippable(stash=["skip"])
    class Stash(nn.Module):
        def forward(self, x):
            yield stash("skip", x)
            return x * 2

    @skippable(pop=["skip"])
    class Pop(nn.Module):
        def forward(self, x):
            s = yield pop("skip")
            return x + s

    def build():
        torch.manual_seed(1)
        return nn.Sequential(nn.Linear(4, 4), Stash(), nn.Linear(4, 4), Pop(), nn.Linear(4, 2))

    ref = build()
    verify_skippables(ref)
    piped = Pipe(build(), balance=[2, 1, 2], devices=["cpu"] * 3, chunks=2, checkpoint="always")
    x = torch.randn(4, 4)
    torch.testing.assert_close(piped(x), ref(x))
    ref(x).sum().backward()
    piped(x).sum().backward()
    for a, b in zip(ref.parameters(), piped.parameters()):
        torch.testing.assert_close(a.grad, b.grad)

    with pytest.raises(TypeError):
        verify_skippables(nn.Sequential(Pop()))
    with pytest.raises(TypeError):
        verify_skippables(nn.Sequential(Stash()))
    ns1, ns2 = Namespace(), Namespace()
    verify_skippables(nn.Sequential(Stash().isolate(ns1), Stash().isolate(ns2), Pop().isolate(ns2), Pop().isolate(ns1)))


def test_block_partition():
    assert blockpartition.solve([1, 2, 3, 4, 5, 6], partitions=2) == [[1, 2, 3, 4], [5, 6]]
    assert blockpartition.solve([6, 5, 4, 3, 2, 1], partitions=3) in ([[6], [5, 4], [3, 2, 1]], [[6], [5], [4, 3, 2, 1]])
    assert balance_cost([1, 1, 1, 1], 4) == [1, 1, 1, 1]
    assert sum(balance_cost([3, 1, 4, 1, 5, 9, 2, 6], 3)) == 8
    with pytest.raises(ValueError):
        blockpartition.solve([1, 2], partitions=3)
