"""Multi-process pipeline, case by case on gloo ranks (cases of the reference's tests/nn/pipe_process/test_pipe.py that apply
to a pipeline whose stages are processes): what each rank holds, constructor checks, batches that do not divide, evaluation
and no-grad runs, a failing layer, lazy construction building only the local layers, ranks without a stage, deferred batch
norm on a stage, and several training steps against the same model trained in one process."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.pipe import AsyncPipe, LazyModule


def _layers(seed=0):
    torch.manual_seed(seed)
    return [nn.Linear(4, 8), nn.Tanh(), nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 2)]


def _step(pipe, rank, last, x, target=None):
    """One forward / backward through all ranks; returns the output on the last stage."""
    out = pipe(x if rank == 0 else None)
    if rank == last:
        loss = out.pow(2).sum() if target is None else nn.functional.mse_loss(out, target)
        loss.backward()
        pipe.back_helper()
        return out
    pipe.back_helper(out)
    return None


def _holdings(rank, world):
    pipe = AsyncPipe(nn.Sequential(*_layers()), balance=[2, 3], chunks=2)
    assert pipe.balance == [2, 3] and pipe.chunks == 2 and pipe.checkpoint == "except_last" and isinstance(pipe.balance, list)
    names = [n for n, _ in pipe.named_parameters()]
    if rank == 0:
        assert len(pipe) == 2 and names == ["partition.0.weight", "partition.0.bias"]
    elif rank == 1:
        assert len(pipe) == 3 and len(names) == 4
    else:
        assert len(pipe) == 0 and names == [] and pipe.partition is None  # more ranks than stages: the rest idle
    # the idle rank takes part in nothing and returns nothing
    out = _step(pipe, rank, 1, torch.randn(4, 4)) if rank < 2 else pipe(None)
    assert (out is not None) == (rank == 1)
    if rank == 2:
        pipe.back_helper()
    dist.barrier()


def test_each_rank_holds_its_stage_and_extra_ranks_idle():
    spawn_ranks(_holdings, 3, (), backend="gloo")


def _constructor_checks(rank, world):
    seq = nn.Sequential(*_layers())
    with pytest.raises(ValueError, match="different length"):
        AsyncPipe(seq, balance=[2, 2])
    with pytest.raises(ValueError, match="positive integer|different length"):
        AsyncPipe(seq, balance=[0, 5])
    with pytest.raises(ValueError, match="chunks must be positive"):
        AsyncPipe(seq, balance=[2, 3], chunks=0)
    with pytest.raises(ValueError, match="checkpoint is not one of"):
        AsyncPipe(seq, balance=[2, 3], checkpoint="sometimes")
    with pytest.raises(IndexError, match="too few ranks"):
        AsyncPipe(seq, balance=[1, 1, 1, 1, 1])
    for mode in ("always", "except_last", "never"):
        AsyncPipe(nn.Sequential(*_layers()), balance=[2, 3], chunks=1, checkpoint=mode)
    dist.barrier()


def test_constructor_checks():
    spawn_ranks(_constructor_checks, 2, (), backend="gloo")


def _batches(rank, world, rows, chunks):
    ref = nn.Sequential(*_layers())
    pipe = AsyncPipe(nn.Sequential(*_layers()), balance=[3, 2], chunks=chunks, checkpoint="always")
    torch.manual_seed(3)
    x = torch.randn(rows, 4)
    out = _step(pipe, rank, 1, x)
    if rank == 1:
        torch.testing.assert_close(out, ref(x))
        assert out.shape == (rows, 2)
    # evaluation: no recomputation, no graph needed
    pipe.eval()
    with torch.no_grad():
        out = pipe(x if rank == 0 else None)
    if rank == 1:
        torch.testing.assert_close(out, ref(x))
        assert not out.requires_grad
    dist.barrier()


@pytest.mark.parametrize("rows,chunks", [(7, 4), (2, 4), (6, 1)])
def test_batches_that_do_not_divide_and_evaluation(rows, chunks):
    spawn_ranks(_batches, 2, (rows, chunks), backend="gloo")


class _Counted(nn.Linear):
    built = 0

    def __init__(self, *a):
        super().__init__(*a)
        type(self).built += 1


def _lazy(rank, world):
    module = [LazyModule(lambda: _Counted(4, 4)), LazyModule(lambda: nn.ReLU()), LazyModule(lambda: _Counted(4, 4)), LazyModule(lambda: _Counted(4, 2))]
    pipe = AsyncPipe(module, balance=[1, 3], chunks=2)
    assert _Counted.built == (1 if rank == 0 else 2)  # only the layers of the local stage were constructed
    assert len(list(pipe.parameters())) == (2 if rank == 0 else 4)
    out = _step(pipe, rank, 1, torch.randn(4, 4))
    assert all(p.grad is not None for p in pipe.parameters())
    assert (out is not None) == (rank == 1)
    dist.barrier()


def _lazy_skippable(rank, world):
    from fairscale_b200.nn.pipe.skip import pop, skippable, stash

    @skippable(stash=["skip"])
    class Stash(nn.Module):
        def forward(self, x):
            yield stash("skip", x)
            return x * 2

    @skippable(pop=["skip"])
    class Pop(nn.Module):
        def forward(self, x):
            skip = yield pop("skip")
            return x + skip

    with pytest.raises(ValueError, match="Skippable layers with multi-process pipe and lazy construction"):
        AsyncPipe([LazyModule(lambda: Stash()), LazyModule(lambda: Pop())], balance=[2], chunks=1)
    # built eagerly and kept inside one stage, the pair works
    pipe = AsyncPipe(nn.Sequential(Stash(), Pop()), balance=[2], chunks=2)
    x = torch.rand(4, 3)
    torch.testing.assert_close(pipe(x), x * 3)


def test_skippable_layers_are_refused_with_lazy_construction():
    spawn_ranks(_lazy_skippable, 1, (), backend="gloo")


def test_lazy_construction_builds_only_the_local_layers():
    spawn_ranks(_lazy, 2, (), backend="gloo")


class _Boom(Exception):
    pass


class _Raise(nn.Module):
    def forward(self, x):
        raise _Boom("layer failed")


def _failing_layer(rank, world):
    """The failure surfaces on the rank that runs the layer; a one-stage pipeline needs nobody else to notice."""
    pipe = AsyncPipe(nn.Sequential(nn.Linear(4, 4), _Raise()), balance=[2], chunks=2)
    if rank == 0:
        with pytest.raises(_Boom):
            pipe(torch.randn(4, 4))
    else:
        assert pipe.partition is None
    dist.barrier()


def test_exception_of_a_layer_surfaces_on_its_rank():
    spawn_ranks(_failing_layer, 2, (), backend="gloo")


def _deferred_batch_norm(rank, world, mode):
    torch.manual_seed(0)
    bn = nn.BatchNorm1d(4)
    layers = [nn.Linear(4, 4), copy.deepcopy(bn), nn.Linear(4, 2)]
    plain = nn.Sequential(*copy.deepcopy(layers))
    pipe = AsyncPipe(nn.Sequential(*layers), balance=[1, 2], chunks=2, checkpoint=mode, deferred_batch_norm=True)
    torch.manual_seed(1)
    x = torch.randn(8, 4)
    _step(pipe, rank, 1, x)
    plain(x).pow(2).sum().backward()
    if rank == 1:
        # running statistics follow the whole mini-batch although the layer saw it in two halves
        torch.testing.assert_close(pipe.partition[0].running_mean, plain[1].running_mean, atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(pipe.partition[0].running_var, plain[1].running_var, atol=1e-2, rtol=1e-2)
        assert int(pipe.partition[0].num_batches_tracked) == 1
    dist.barrier()


@pytest.mark.parametrize("mode", ["never", "always"])
def test_deferred_batch_norm_on_a_stage(mode):
    spawn_ranks(_deferred_batch_norm, 2, (mode,), backend="gloo")


def _training(rank, world, mode):
    """Five optimizer steps: every stage ends with the weights the one-process model has."""
    balance = [2, 1, 2]
    plain = nn.Sequential(*_layers())
    pipe = AsyncPipe(nn.Sequential(*_layers()), balance=balance, chunks=3, checkpoint=mode)
    opt = torch.optim.SGD(pipe.parameters(), lr=0.1, momentum=0.9)
    plain_opt = torch.optim.SGD(plain.parameters(), lr=0.1, momentum=0.9)
    g = torch.Generator().manual_seed(7)
    for _ in range(5):
        x, y = torch.randn(6, 4, generator=g), torch.randn(6, 2, generator=g)
        opt.zero_grad()
        _step(pipe, rank, 2, x, y)
        opt.step()
        plain_opt.zero_grad()
        nn.functional.mse_loss(plain(x), y).backward()
        plain_opt.step()
    lo = sum(balance[:rank])
    mine = [p for layer in list(plain)[lo: lo + balance[rank]] for p in layer.parameters()]
    assert len(mine) == len(list(pipe.parameters()))
    for a, b in zip(pipe.parameters(), mine):
        torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-4)
    dist.barrier()


@pytest.mark.parametrize("mode", ["never", "except_last", "always"])
def test_training_matches_the_one_process_model(mode):
    spawn_ranks(_training, 3, (mode,), backend="gloo")
