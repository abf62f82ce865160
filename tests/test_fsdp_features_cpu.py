"""FSDP behaviours beyond plain training parity (2 gloo ranks, CPU): ``apply`` on sharded weights, frozen sub-modules,
two forwards before two backwards, a module called several times per step, nesting with ``checkpoint_wrapper``,
``summon_full_params`` variants, input casting under mixed precision, evaluation without gradients."""
import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn import FullyShardedDataParallel as FSDP
from fairscale_b200.nn import checkpoint_wrapper
from fairscale_b200.nn.data_parallel import TrainingState, get_fsdp_instances

CPU = dict(compute_device=torch.device("cpu"))


def _mlp(d=8, seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(d, 2 * d + 1), nn.ReLU(), nn.Linear(2 * d + 1, d), nn.ReLU(), nn.Linear(d, 4))


def _x(rank, step, d=8):
    g = torch.Generator().manual_seed(31 * step + rank)
    return torch.randn(5, d, generator=g)


def _wrap(model, **kw):
    layers = list(model)
    return FSDP(nn.Sequential(FSDP(nn.Sequential(*layers[:2]), **CPU, **kw), *layers[2:]), **CPU, **kw)


def _assert_same_as_ddp(model, ref):
    full, ref_sd = model.state_dict(), ref.module.state_dict()
    assert len(full) == len(ref_sd)
    for v, w in zip(full.values(), ref_sd.values()):  # names differ by the wrapper nesting, the order does not
        torch.testing.assert_close(v, w, atol=1e-6, rtol=1e-5)


def _apply_and_freeze(rank, world):
    # apply(): the function sees full (unsharded) parameters and its writes survive resharding
    model = _wrap(_mlp())

    def init(m):
        if isinstance(m, nn.Linear):
            with torch.no_grad():
                m.weight.fill_(0.25)
                m.bias.zero_()

    model.apply(init)
    sd = model.state_dict()
    assert all(torch.all(v == (0.25 if k.endswith("weight") else 0.0)) for k, v in sd.items())

    # frozen inner unit: its shard never changes, the trainable part matches DDP with the same freezing
    ref_m = _mlp()
    for p in list(ref_m[0].parameters()):
        p.requires_grad = False
    ref = nn.parallel.DistributedDataParallel(ref_m)
    ref_opt = torch.optim.SGD([p for p in ref.parameters() if p.requires_grad], lr=0.1)
    base = _mlp()
    for p in list(base[0].parameters()):
        p.requires_grad = False
    model = _wrap(base)
    opt = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=0.1)
    for s in range(3):
        for m, o in ((ref, ref_opt), (model, opt)):
            o.zero_grad()
            m(_x(rank, s)).pow(2).mean().backward()
            o.step()
    _assert_same_as_ddp(model, ref)
    for inst in get_fsdp_instances(model):
        assert inst.training_state == TrainingState.IDLE


def test_fsdp_apply_and_frozen_unit():
    spawn_ranks(_apply_and_freeze, 2, (), backend="gloo")


class _ManualDP:
    """Oracle for gradient patterns DDP's reducer does not support (several forwards before the backwards): a bare
    replica whose accumulated local gradients are averaged by hand before the optimizer step."""

    def __init__(self, model):
        self.module = model

    def __call__(self, x):
        return self.module(x)

    def parameters(self):
        return self.module.parameters()

    def average_grads(self, world):
        for p in self.module.parameters():
            dist.all_reduce(p.grad)
            p.grad /= world


def _multi_forward(rank, world):
    ref = _ManualDP(_mlp())
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    model = _wrap(_mlp())
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    # two forwards, then the two backwards (the first graph outlives the second forward); both backwards reduce
    for m, o in ((ref, ref_opt), (model, opt)):
        o.zero_grad()
        l1 = m(_x(rank, 0)).pow(2).mean()
        l2 = m(_x(rank, 1)).pow(2).mean()
        l1.backward()
        l2.backward()
        if m is ref:
            ref.average_grads(world)
        o.step()
    _assert_same_as_ddp(model, ref)
    # the same with only the last backward reducing
    for m, o in ((ref, ref_opt), (model, opt)):
        o.zero_grad()
        l1 = m(_x(rank, 4)).pow(2).mean()
        l2 = m(_x(rank, 5)).pow(2).mean()
        if m is ref:
            l1.backward()
            l2.backward()
            ref.average_grads(world)
        else:
            with model.no_sync():
                l1.backward()
            l2.backward()
        o.step()
    _assert_same_as_ddp(model, ref)
    # one summed loss over two forwards of the same wrapper
    for m, o in ((ref, ref_opt), (model, opt)):
        o.zero_grad()
        (m(_x(rank, 2)).pow(2).mean() + m(_x(rank, 3)).abs().mean()).backward()
        if m is ref:
            ref.average_grads(world)
        o.step()
    _assert_same_as_ddp(model, ref)


def test_fsdp_forward_forward_backward_backward():
    spawn_ranks(_multi_forward, 2, (), backend="gloo")


def _with_checkpoint(rank, world):
    ref = nn.parallel.DistributedDataParallel(_mlp())
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    layers = list(_mlp())
    # both nestings: FSDP(checkpoint(m)) and checkpoint(FSDP(m))
    a = FSDP(checkpoint_wrapper(nn.Sequential(*layers[:2])), **CPU)
    b = checkpoint_wrapper(FSDP(nn.Sequential(*layers[2:4]), **CPU))
    model = FSDP(nn.Sequential(a, b, layers[4]), **CPU)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    for s in range(3):
        losses = []
        for m, o in ((ref, ref_opt), (model, opt)):
            o.zero_grad()
            x = _x(rank, s).requires_grad_()
            loss = m(x).pow(2).mean()
            loss.backward()
            o.step()
            losses.append(loss.item())
        assert abs(losses[0] - losses[1]) < 1e-6
    full = model.state_dict()
    ref_sd = ref.module.state_dict()
    assert len(full) == len(ref_sd)
    for v, w in zip(full.values(), ref_sd.values()):  # names differ by the wrapper nesting, the order does not
        torch.testing.assert_close(v, w, atol=1e-6, rtol=1e-5)


def test_fsdp_with_checkpoint_wrapper_both_nestings():
    spawn_ranks(_with_checkpoint, 2, (), backend="gloo")


def _summon_eval_inputs(rank, world):
    model = _wrap(_mlp())
    before = model.state_dict()
    # volatile: modifications are discarded
    with model.summon_full_params(volatile=True):
        with torch.no_grad():
            for p in model.parameters():
                p.add_(1.0)
    after = model.state_dict()
    for k in before:
        torch.testing.assert_close(after[k], before[k])
    # recurse=False only gathers the outer unit
    with model.summon_full_params(recurse=False):
        outer_full = [p.numel() for p in model.params]
    assert sum(outer_full) == sum(p.numel() for p in list(_mlp())[2:] for p in p.parameters())
    # evaluation under no_grad leaves every unit idle and resharded
    model.eval()
    with torch.no_grad():
        y1 = model(_x(rank, 0))
        y2 = model(_x(rank, 0))
    torch.testing.assert_close(y1, y2)
    for inst in get_fsdp_instances(model):
        assert inst.training_state == TrainingState.IDLE
    # mixed precision: fp32 inputs are cast to the compute dtype at the root, integer inputs pass through
    mp = FSDP(_mlp(), mixed_precision=True, compute_dtype=torch.bfloat16, **CPU)
    out = mp(_x(rank, 0))
    assert out.dtype == torch.bfloat16
    out.float().sum().backward()
    assert mp.params[0].grad is not None and mp.params[0].grad.dtype == torch.float32
    emb = FSDP(nn.Sequential(nn.Embedding(10, 8), nn.Linear(8, 2)), mixed_precision=True, compute_dtype=torch.bfloat16, **CPU)
    assert emb(torch.randint(0, 10, (3, 4))).dtype == torch.bfloat16
    dist.barrier()


def test_fsdp_summon_eval_and_input_casting():
    spawn_ranks(_summon_eval_inputs, 2, (), backend="gloo")


class _Shared(nn.Module):
    """Four linears; l1 and l3 share the weight or the bias (each keeps one parameter of its own)."""

    def __init__(self, sharing, with_fsdp=False, inner_flat=False):
        super().__init__()
        torch.manual_seed(2)
        self.l0, self.l1, self.l2, self.l3 = (nn.Linear(4, 4) for _ in range(4))
        if sharing == "weight":
            self.l1.weight = self.l3.weight
        elif sharing == "bias":
            self.l1.bias = self.l3.bias
        if with_fsdp:
            self.l1 = FSDP(self.l1, flatten_parameters=False, **CPU)  # units that share parameters stay unflattened
            self.l2 = FSDP(self.l2, flatten_parameters=inner_flat, **CPU)
            self.l3 = FSDP(self.l3, flatten_parameters=False, **CPU)
            if sharing == "weight":
                self.l3.append_shared_param(self.l1.module.weight)
            elif sharing == "bias":
                self.l3.append_shared_param(self.l1.module.bias)

    def forward(self, x):
        return self.l3(self.l2(self.l1(self.l0(x))))


def _shared_weights(rank, world, sharing, inner_flat):
    ref = nn.parallel.DistributedDataParallel(_Shared(sharing))
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    model = FSDP(_Shared(sharing, with_fsdp=True, inner_flat=inner_flat), flatten_parameters=False, **CPU)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    for s in range(3):
        for m, o in ((ref, ref_opt), (model, opt)):
            o.zero_grad()
            m(_x(rank, s, d=4)).pow(2).mean().backward()
            o.step()
    full, ref_sd = model.state_dict(), ref.module.state_dict()
    assert set(full) == set(ref_sd)
    for k in ref_sd:
        torch.testing.assert_close(full[k], ref_sd[k], atol=1e-6, rtol=1e-5)
    if sharing == "weight":
        torch.testing.assert_close(full["l1.weight"], full["l3.weight"])


@pytest.mark.parametrize("sharing,inner_flat", [("weight", False), ("bias", True), (None, True)])
def test_fsdp_units_sharing_a_parameter(sharing, inner_flat):
    spawn_ranks(_shared_weights, 2, (sharing, inner_flat), backend="gloo")


def _rewrap(rank, world):
    # wrap, train, take the bare module back out, wrap it again with other settings: the weights carry over
    inner = _mlp()
    first = FSDP(inner, flatten_parameters=True, **CPU)
    opt = torch.optim.SGD(first.parameters(), lr=0.1)
    first(_x(rank, 0)).pow(2).mean().backward()
    opt.step()
    trained = first.state_dict()
    with first.summon_full_params():
        bare = _mlp()
        bare.load_state_dict(first.module.state_dict() if not hasattr(first.module, "module") else first.module.module.state_dict())
    second = FSDP(bare, flatten_parameters=False, reshard_after_forward=False, **CPU)
    again = second.state_dict()
    for k in trained:
        torch.testing.assert_close(again[k], trained[k])
    second(_x(rank, 1)).pow(2).mean().backward()
    assert all(p.grad is not None for p in second.params)


def test_fsdp_wrap_unwrap_wrap_again():
    spawn_ranks(_rewrap, 2, (), backend="gloo")


class _TiedVocab(nn.Module):
    """Embedding and a memory-efficient vocabulary output layer that share one weight, each in its own FSDP unit."""

    def __init__(self, with_fsdp):
        super().__init__()
        from fairscale_b200.experimental.nn import MEVO

        torch.manual_seed(4)
        self.l0 = nn.Embedding(12, 8)
        nn.init.uniform_(self.l0.weight, -0.1, 0.1)
        self.l1 = MEVO(self.l0.weight, tile_factor=2, reduction="sum")
        self.middle = nn.Linear(8, 8)
        self.ln1, self.ln2 = nn.LayerNorm(8), nn.LayerNorm(8)
        if with_fsdp:
            self.l0 = FSDP(self.l0, flatten_parameters=False, **CPU)
            self.l1 = FSDP(self.l1, flatten_parameters=False, **CPU)
            self.l1.append_shared_param(self.l0.module.weight)

    def forward(self, tokens):
        target = (tokens + 1) % 12
        x = self.ln2(self.middle(self.ln1(self.l0(tokens))))
        return self.l1(x, target)


def _tied_vocab(rank, world):
    ref = nn.parallel.DistributedDataParallel(_TiedVocab(False))
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    model = FSDP(_TiedVocab(True), flatten_parameters=False, **CPU)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(rank)
    tokens = torch.randint(0, 12, (3, 5), generator=g)
    for _ in range(3):
        losses = []
        for m, o in ((ref, ref_opt), (model, opt)):
            o.zero_grad()
            loss = m(tokens)
            loss.backward()
            o.step()
            losses.append(loss.item())
        assert abs(losses[0] - losses[1]) < 1e-4 * max(1.0, abs(losses[0]))
    full, ref_sd = model.state_dict(), ref.module.state_dict()
    torch.testing.assert_close(full["l0.weight"], ref_sd["l0.weight"], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(full["middle.weight"], ref_sd["middle.weight"], atol=1e-5, rtol=1e-4)


def test_fsdp_embedding_and_mevo_output_share_a_weight():
    spawn_ranks(_tied_vocab, 2, (), backend="gloo")


class _TwoHeads(nn.Module):
    """Returns a tuple that contains one tensor twice plus a second head: the pre-backward work must run once."""

    def __init__(self):
        super().__init__()
        torch.manual_seed(6)
        self.body = nn.Linear(8, 8)
        self.head = nn.Linear(8, 2)

    def forward(self, x):
        h = torch.tanh(self.body(x))
        return h, h, self.head(h)


def _outputs_and_reuse(rank, world):
    # (a) several outputs, one of them twice, losses on all of them
    ref = nn.parallel.DistributedDataParallel(_TwoHeads())
    model = FSDP(_TwoHeads(), **CPU)
    calls = []
    orig = model._prep_grads_for_backward
    model._prep_grads_for_backward = lambda: (calls.append(1), orig())[1]
    for m in (ref, model):
        a, b, c = m(_x(rank, 0))
        (a.sum() + 2 * b.sum() + c.pow(2).sum()).backward()
    assert len(calls) == 1  # one preparation of the gradients per backward, however many outputs carry a hook
    flat_ref = torch.cat([p.grad.reshape(-1) for p in ref.module.parameters()])
    g = model.params[0].grad
    parts = [torch.zeros_like(g) for _ in range(world)]
    dist.all_gather(parts, g)
    torch.testing.assert_close(torch.cat(parts)[: flat_ref.numel()], flat_ref, atol=1e-6, rtol=1e-5)

    # (b) one checkpointed FSDP unit called twice inside a forward
    torch.manual_seed(7)
    blk = nn.Sequential(nn.Linear(8, 8), nn.Tanh())
    tail = nn.Linear(8, 3)
    import copy

    ref_blk, ref_tail = copy.deepcopy(blk), copy.deepcopy(tail)

    class Twice(nn.Module):
        def __init__(self, b, t):
            super().__init__()
            self.b, self.t = b, t

        def forward(self, x):
            return self.t(self.b(self.b(x)))

    ref2 = nn.parallel.DistributedDataParallel(Twice(ref_blk, ref_tail))
    model2 = FSDP(Twice(FSDP(checkpoint_wrapper(blk), **CPU), tail), **CPU)
    for m in (ref2, model2):
        m(_x(rank, 1).requires_grad_()).pow(2).mean().backward()
    inner = model2.module.b
    gref = torch.cat([p.grad.reshape(-1) for p in ref_blk.parameters()])
    g = inner.params[0].grad
    parts = [torch.zeros_like(g) for _ in range(world)]
    dist.all_gather(parts, g)
    torch.testing.assert_close(torch.cat(parts)[: gref.numel()], gref, atol=1e-6, rtol=1e-5)

    # (c) full state dict only on rank 0
    model3 = FSDP(_mlp(), state_dict_on_rank_0_only=True, **CPU)
    sd = model3.state_dict()
    assert (len(sd) > 0) == (rank == 0)


def test_fsdp_multiple_outputs_module_reuse_and_rank0_state_dict():
    spawn_ranks(_outputs_and_reuse, 2, (), backend="gloo")


def _conv_bn(rank, world):
    """A small conv net whose BatchNorm layers get their own fp32 FSDP wrappers (auto_wrap_bn); the rest trains in one
    mixed-precision unit.  Every rank sees the same batch, so local BatchNorm statistics equal DDP's."""
    from fairscale_b200.nn.data_parallel import auto_wrap_bn

    def net():
        torch.manual_seed(8)
        return nn.Sequential(nn.Conv2d(2, 4, 3, padding=1), nn.BatchNorm2d(4), nn.ReLU(), nn.Conv2d(4, 4, 3, padding=1), nn.BatchNorm2d(4),
                             nn.ReLU(), nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(4, 3))

    ref = nn.parallel.DistributedDataParallel(net())
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    wrapped = auto_wrap_bn(net(), single_rank_pg=False, fsdp_config={"mixed_precision": False, "flatten_parameters": False,
                                                                      "reshard_after_forward": False, "bucket_cap_mb": 0,
                                                                      "compute_device": torch.device("cpu")})
    n_bn = sum(isinstance(m, FSDP) for m in wrapped.modules())
    assert n_bn == 2 and all(isinstance(m.module.module if hasattr(m.module, "module") else m.module, nn.BatchNorm2d)
                             for m in wrapped.modules() if isinstance(m, FSDP))
    model = FSDP(wrapped, **CPU)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 2, 5, 5, generator=g)
    for _ in range(3):
        for m, o in ((ref, ref_opt), (model, opt)):
            o.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    full, ref_sd = model.state_dict(), ref.module.state_dict()
    assert set(full) == set(ref_sd)
    for k in ref_sd:
        torch.testing.assert_close(full[k].float(), ref_sd[k].float(), atol=1e-5, rtol=1e-4)


def test_fsdp_auto_wrap_bn_conv_net():
    spawn_ranks(_conv_bn, 2, (), backend="gloo")


def _state_dict_properties(rank, world):
    torch.manual_seed(9)
    net = nn.Sequential(nn.Linear(8, 8), nn.BatchNorm1d(8), nn.Linear(8, 3))
    model = FSDP(net, mixed_precision=True, compute_dtype=torch.bfloat16, state_dict_device=torch.device("cpu"), **CPU)
    model(_x(rank, 0)).float().sum().backward()
    sd = model.state_dict()
    # full precision parameters under the bare module's names, buffers included, on the requested device
    assert {"0.weight", "1.running_mean", "1.num_batches_tracked", "2.bias"} <= set(sd)
    assert all(v.dtype == torch.float32 for k, v in sd.items() if v.is_floating_point())
    assert all(v.device.type == "cpu" for v in sd.values())
    # strict loading: an unexpected key is refused, the exact dict loads, values survive the round trip
    bad = dict(sd)
    bad["nope"] = torch.zeros(1)
    with pytest.raises(RuntimeError):
        model.load_state_dict(bad, strict=True)
    changed = {k: (v + 1 if v.is_floating_point() else v) for k, v in sd.items()}
    model.load_state_dict(changed)
    again = model.state_dict()
    for k, v in changed.items():
        if "running_" in k:  # buffers live in the compute dtype under mixed precision (buffer_dtype=None), as in the reference
            torch.testing.assert_close(again[k], v, atol=2e-2, rtol=2e-2)
        else:
            torch.testing.assert_close(again[k], v)  # parameters come back from the fp32 master shards unchanged
    # state dict of a model in eval mode, taken under no_grad, is the same object graph-free
    model.eval()
    with torch.no_grad():
        assert all(not v.requires_grad for v in model.state_dict().values())


def test_fsdp_state_dict_dtype_device_and_strictness():
    spawn_ranks(_state_dict_properties, 2, (), backend="gloo")


def _collective_counts(rank, world, reshard):
    """One forward + backward issues an all-gather per unit in forward and, when units are resharded after forward,
    one more per non-root unit in backward (2 n - 1 in total, as the reference's test_fsdp_grad_acc counts); one
    reduce-scatter per unit, none under no_sync."""
    from fairscale_b200.parallel import comm

    kw = dict(reshard_after_forward=reshard, bucket_cap_mb=0, **CPU)
    layers = list(_mlp())
    model = FSDP(nn.Sequential(FSDP(nn.Sequential(*layers[:2]), **kw), FSDP(nn.Sequential(*layers[2:4]), **kw), layers[4]), **kw)
    n = len(get_fsdp_instances(model))
    assert n == 3
    model(_x(rank, 0)).sum().backward()  # first pass also records the execution order
    comm.reset_counters()
    model(_x(rank, 1)).sum().backward()
    c = comm.counters()
    assert c["all_gather"] == (2 * n - 1 if reshard else n), c
    assert c["reduce_scatter"] == n, c
    comm.reset_counters()
    with model.no_sync():
        model(_x(rank, 2)).sum().backward()
    c = comm.counters()
    assert c["reduce_scatter"] == 0 and c["all_gather"] >= n, c


@pytest.mark.parametrize("reshard", [True, False])
def test_fsdp_number_of_collectives_per_step(reshard):
    spawn_ranks(_collective_counts, 2, (reshard,), backend="gloo")


class _DictIn(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(3)
        self.lin = nn.Linear(4, 4)

    def forward(self, batch, scale=None, extra=None):
        x = batch["x"] if isinstance(batch, dict) else batch[0]
        y = self.lin(x)
        if scale is not None:
            y = y * scale
        assert extra is None or extra == "tag"
        return {"out": y, "ids": batch["ids"] if isinstance(batch, dict) else None}


def _inputs(rank, world):
    # containers in, containers out; floating inputs are cast to the compute dtype, integer ones and strings pass through
    model = FSDP(_DictIn(), mixed_precision=True, compute_dtype=torch.bfloat16, **CPU)
    ids = torch.arange(3)
    out = model({"x": torch.randn(3, 4), "ids": ids}, scale=torch.tensor(2.0), extra="tag")
    assert out["out"].dtype == torch.bfloat16 and out["ids"].dtype == torch.int64 and torch.equal(out["ids"], ids)
    out["out"].float().sum().backward()
    assert model.params[0].grad is not None
    out = model([torch.randn(3, 4)])
    assert out["out"].shape == (3, 4) and out["ids"] is None
    # full precision: inputs are left alone
    fp32 = FSDP(_DictIn(), **CPU)
    assert fp32({"x": torch.randn(3, 4), "ids": ids})["out"].dtype == torch.float32


def test_fsdp_container_inputs_and_casting():
    spawn_ranks(_inputs, 2, (), backend="gloo")
