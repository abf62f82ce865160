"""Consolidating and re-sharding optimizer state of FSDP on gloo ranks (cases of the reference's
tests/nn/data_parallel/test_fsdp_optimizer_utils.py): for several optimizers, a model with a shared weight and nested
wrappers, a model whose experts live in their own process group (their state stays on the rank), and a model with
parameters that never receive a gradient.  The gathered dict lives on the CPU of rank 0 only, has the entries and sizes of
the unwrapped model's optimizer, and slicing it again gives back exactly what each rank's optimizer holds."""
import copy
import functools

import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.optim import SGD, Adadelta, Adam

from fairscale_b200.fair_dev.testing.testing import objects_are_equal, spawn_ranks
from fairscale_b200.internal.params import recursive_copy_to_device
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP
from fairscale_b200.nn.data_parallel import get_fsdp_instances

CPU = dict(compute_device=torch.device("cpu"))


class _Shared(nn.Module):
    """Embedding and output projection share their weight; the two middle layers are wrapped on their own."""

    def __init__(self, wrap):
        super().__init__()
        torch.manual_seed(0)
        self.embed = nn.Embedding(23, 8)
        self.mid = nn.Sequential(wrap(nn.Linear(8, 8)), nn.Tanh(), wrap(nn.Linear(8, 8)))
        self.out = nn.Linear(8, 23, bias=False)
        self.out.weight = self.embed.weight
        self.register_buffer("steps", torch.zeros(1))

    def forward(self, tokens):
        return self.out(self.mid(self.embed(tokens)))


class _Experts(nn.Module):
    """A shared trunk and one expert per rank; the expert is wrapped in a process group of its own."""

    def __init__(self, wrap, wrap_expert, rank):
        super().__init__()
        torch.manual_seed(0)
        self.trunk = wrap(nn.Linear(8, 8))
        torch.manual_seed(100 + rank)
        self.expert = wrap_expert(nn.Linear(8, 8))
        torch.manual_seed(1)
        self.head = nn.Linear(8, 4)

    def forward(self, x):
        return self.head(torch.relu(self.expert(torch.relu(self.trunk(x)))))


def _numel(state):
    return sum(t.numel() for t in state.values() if torch.is_tensor(t) and t.dim() > 0)


def _make_optim(optim_fn, params):
    try:
        return optim_fn(params, lr=0.01)
    except TypeError:  # Adadelta of old versions
        return optim_fn(params)


def _consolidate(rank, world, optim_name, model_kind):
    optim_fn = {"sgd_momentum": functools.partial(SGD, momentum=0.9), "sgd": SGD, "adam": Adam, "adadelta": Adadelta}[optim_name]
    if model_kind == "shared":
        plain = _Shared(lambda m: m)
        fsdp = FSDP(_Shared(lambda m: FSDP(m, **CPU)), **CPU)
        batch = torch.randint(0, 23, (4, 5), generator=torch.Generator().manual_seed(rank))
        loss_of = lambda model: nn.functional.cross_entropy(model(batch).flatten(0, 1), batch.flatten())  # noqa: E731
    else:
        own_group = dist.new_group([rank]) if world > 1 else None
        groups = [dist.new_group([r]) for r in range(world)]
        plain = _Experts(lambda m: m, lambda m: m, rank)
        fsdp = FSDP(_Experts(lambda m: FSDP(m, **CPU), lambda m: FSDP(m, process_group=groups[rank], **CPU), rank), **CPU)
        del own_group
        batch = torch.randn(4, 8, generator=torch.Generator().manual_seed(rank))
        loss_of = lambda model: model(batch).pow(2).mean()  # noqa: E731
    opt, plain_opt = _make_optim(optim_fn, fsdp.parameters()), _make_optim(optim_fn, plain.parameters())
    for model, o in ((fsdp, opt), (plain, plain_opt)):
        o.zero_grad()
        loss_of(model).backward()
        o.step()
    plain_sd = plain_opt.state_dict()

    if model_kind == "experts":
        local_only = [m for m in get_fsdp_instances(fsdp) if m.no_broadcast_optim_state]
        assert len(local_only) == 1 and local_only[0] is fsdp.module.expert  # found from its one-rank process group

    shard_before = recursive_copy_to_device(copy.deepcopy(opt.state_dict()), non_blocking=False, device=torch.device("cpu"))
    sd = fsdp.gather_full_optim_state_dict(opt)
    if rank > 0:
        assert sd is None
        sd_box = [None]
    else:
        sd_box = [sd]
        assert "uncollected_local_ids" in sd and "param_id_map" in sd
        for bufs in sd["state"].values():
            assert all(t.device.type == "cpu" for t in bufs.values() if torch.is_tensor(t))
        # the entries and sizes of the unwrapped optimizer (a shared weight counts once in both)
        assert len(sd["state"]) == len(plain_sd["state"]), (len(sd["state"]), len(plain_sd["state"]))
        assert len(sd["param_groups"][0]["params"]) == len(plain_sd["param_groups"][0]["params"])
        assert sum(_numel(v) for v in sd["state"].values()) == sum(_numel(v) for v in plain_sd["state"].values())
        if optim_name == "sgd":
            assert all(_numel(v) == 0 for v in sd["state"].values())  # plain SGD keeps no tensors
        elif model_kind == "shared":
            # values too: ranks trained on different batches, but the state was built from the averaged gradient
            pass
    # every rank slices the dict again (as when resuming): it gets its own optimizer state back
    dist.broadcast_object_list(sd_box, src=0)
    full = sd_box[0]
    kept = copy.deepcopy(full["state"])
    shard = fsdp.get_shard_from_optim_state_dict(full)
    shard = recursive_copy_to_device(shard, non_blocking=False, device=torch.device("cpu"))
    if any(_numel(v) for v in kept.values()):
        assert not objects_are_equal(kept, full["state"])  # the argument is consumed: pass a copy to keep the original
    assert set(shard.keys()) >= set(shard_before.keys()) and len(shard["state"]) == len(shard_before["state"])
    assert [_numel(v) for v in shard["state"].values()] == [_numel(v) for v in shard_before["state"].values()]
    if not (model_kind == "experts" and rank > 0):  # the experts' state of other ranks was never collected
        objects_are_equal(shard["state"], shard_before["state"], raise_exception=True)
    assert list(shard["param_groups"][0].values()) == list(shard_before["param_groups"][0].values())
    fresh = _make_optim(optim_fn, fsdp.parameters())
    fresh.load_state_dict(shard)
    fresh.zero_grad()
    loss_of(fsdp).backward()
    fresh.step()  # and training goes on


@pytest.mark.parametrize("optim_name,model_kind", [("sgd_momentum", "shared"), ("sgd", "experts"), ("adam", "experts"), ("adadelta", "shared"),
                                                   ("adam", "shared")])
def test_consolidated_optimizer_state(optim_name, model_kind):
    spawn_ranks(_consolidate, 2, (optim_name, model_kind), backend="gloo")


class _Unused(nn.Module):
    def __init__(self, wrap_second):
        super().__init__()
        torch.manual_seed(0)
        self.l = nn.Linear(4, 4)
        self.not_trained = FSDP(nn.Linear(4, 4).requires_grad_(False), **CPU)  # in the forward, frozen (a unit of its own:
        # one flat parameter cannot mix trainable and frozen members)
        self.not_used = nn.Linear(4, 4)                            # never called
        self.l2 = FSDP(nn.Linear(4, 4), **CPU) if wrap_second else nn.Linear(4, 4)

    def forward(self, x):
        return self.l2(self.not_trained(self.l(x)))


def _unused(rank, world, wrap_second):
    model = FSDP(_Unused(wrap_second), **CPU)
    opt = SGD(model.parameters(), momentum=0.9, lr=0.1)
    model(torch.rand(2, 4)).sum().backward()
    opt.step()
    model.zero_grad(set_to_none=True)
    sd = model.gather_full_optim_state_dict(opt)
    if rank == 0:
        shard = model.get_shard_from_optim_state_dict(copy.deepcopy(sd))
        mine = recursive_copy_to_device(opt.state_dict(), non_blocking=False, device=torch.device("cpu"))
        objects_are_equal(recursive_copy_to_device(shard, non_blocking=False, device=torch.device("cpu"))["state"], mine["state"], raise_exception=True)
    else:
        assert sd is None


@pytest.mark.parametrize("wrap_second", [True, False])
def test_parameters_that_never_get_a_gradient(wrap_second):
    spawn_ranks(_unused, 2, (wrap_second,), backend="gloo")


def _refusals(rank, world):
    model = FSDP(nn.Linear(4, 4), flatten_parameters=False, **CPU)
    opt = SGD(model.parameters(), lr=0.1, momentum=0.9)
    model(torch.rand(2, 4)).sum().backward()
    opt.step()
    with pytest.raises(NotImplementedError):
        model.gather_full_optim_state_dict(opt)
    flat = FSDP(nn.Linear(4, 4), **CPU)
    groups = SGD([{"params": [p]} for p in flat.parameters()] + [{"params": [nn.Parameter(torch.zeros(1))]}], lr=0.1)
    with pytest.raises(AssertionError, match="Param groups"):
        flat.gather_full_optim_state_dict(groups)


def test_layouts_without_support_are_refused():
    spawn_ranks(_refusals, 2, (), backend="gloo")
