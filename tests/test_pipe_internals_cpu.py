"""The small parts the GPipe scheduler is made of (single process, CPU): phony tensors, fork / join dependencies,
micro-batches, CPU streams, worker threads, portals and skip bookkeeping, skippable verification, leaks."""
import gc
import weakref

import pytest
import torch
from torch import nn

from fairscale_b200.nn.pipe import Pipe
from fairscale_b200.nn.pipe import microbatch
from fairscale_b200.nn.pipe.dependency import fork, join
from fairscale_b200.nn.pipe.phony import get_phony
from fairscale_b200.nn.pipe.skip import Namespace, pop, skippable, stash, verify_skippables
from fairscale_b200.nn.pipe.skip.layout import inspect_skip_layout
from fairscale_b200.nn.pipe.skip.tracker import StageSkipTracker
from fairscale_b200.nn.pipe.stream import CPUStream, current_stream, default_stream, get_device, is_cuda, new_stream, use_stream, wait_stream
from fairscale_b200.nn.pipe.worker import Task, spawn_workers

CPU = torch.device("cpu")


def test_phony_is_cached_per_device_and_flag():
    a, b = get_phony(CPU, requires_grad=True), get_phony(CPU, requires_grad=True)
    c = get_phony(CPU, requires_grad=False)
    assert a is b and a is not c
    assert a.numel() == 0 and a.requires_grad and not c.requires_grad


def test_fork_join_orders_backward():
    order = []

    class Log(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, tag):
            ctx.tag = tag
            return x.clone()

        @staticmethod
        def backward(ctx, g):
            order.append(ctx.tag)
            return g, None

    a = torch.ones(1, requires_grad=True)
    b = torch.ones(1, requires_grad=True)
    x = Log.apply(a, "a")
    y = Log.apply(b, "b")
    # the phony edge from x into y's branch makes backward finish y's branch ("b") before it reaches x's producer ("a")
    x, phony = fork(x)
    y = join(y, phony)
    assert phony.numel() == 0
    (x + y).sum().backward()
    assert sorted(order) == ["a", "b"] and order.index("b") < order.index("a")
    assert torch.equal(a.grad, torch.ones(1)) and torch.equal(b.grad, torch.ones(1))
    # without grad there is nothing to tie
    with torch.no_grad():
        x2, p2 = fork(torch.ones(1))
        assert join(torch.ones(1), p2).requires_grad is False


def test_microbatch_scatter_gather_and_checks():
    x = torch.arange(10.0).view(5, 2)
    parts = microbatch.scatter(x, chunks=3)
    assert [p.tensor.shape[0] for p in parts] == [2, 2, 1] and [p.index for p in parts] == [0, 1, 2]
    assert torch.equal(microbatch.gather(parts), x)
    pair = microbatch.scatter((x, x * 2), chunks=2)
    assert len(pair) == 2 and len(pair[0]) == 2
    out = microbatch.gather(pair)
    assert isinstance(out, tuple) and torch.equal(out[1], x * 2)
    doubled = parts[0].call(lambda t: t * 2)
    assert torch.equal(doubled.tensor, parts[0].tensor * 2) and doubled.index == 0
    with pytest.raises(TypeError):
        microbatch.check("not a tensor")
    with pytest.raises(TypeError):
        microbatch.check((x, 1))


def test_cpu_streams_are_inert():
    s = new_stream(CPU)
    assert s is CPUStream and current_stream(CPU) is CPUStream and default_stream(CPU) is CPUStream
    assert not is_cuda(s) and get_device(s) == CPU
    with use_stream(s):
        wait_stream(s, s)


def test_worker_threads_run_tasks_and_forward_exceptions():
    with spawn_workers([CPU, CPU]) as (in_queues, out_queues):
        assert len(in_queues) == 2
        batch = microbatch.Batch(torch.ones(2), 0)
        in_queues[0].put(Task(CPUStream, compute=lambda: batch.call(lambda t: t + 1), finalize=None))
        ok, payload = out_queues[0].get()
        assert ok
        task, result = payload
        assert torch.equal(result.tensor, torch.full((2,), 2.0))

        def boom():
            raise ValueError("from the worker")

        in_queues[1].put(Task(CPUStream, compute=boom, finalize=None))
        ok, payload = out_queues[1].get()
        assert not ok and payload[0] is ValueError


def test_routed_skip_tensors_travel_as_stage_ports():
    """A skip tensor that crosses partitions is stashed into the stage's outbox, waits in transit, is moved by ``copy``
    and comes back through ``deliver`` as an extra stage input; its gradient flows through those nodes."""
    Stash, Pop = _skip_model()
    parts = [nn.Sequential(Stash()), nn.Sequential(nn.Identity()), nn.Sequential(Pop())]
    layout = inspect_skip_layout(parts)
    (key,) = layout.exports(0)
    assert layout.imports(2) == [key] and layout.imports(1) == [] and layout.exports(2) == []
    tracker = StageSkipTracker(layout, index=3)
    assert tracker.index == 3
    src = torch.ones(3, requires_grad=True)
    carrier = microbatch.Batch(torch.zeros(1), 3)
    tracker.save(carrier, key[0], key[1], src * 3)      # routed: goes to the outbox, not into the dictionary
    assert key in tracker.outbox and not tracker.tensors
    tracker.in_transit[key] = tracker.outbox.pop(key)   # what the pipeline does after the stage has run
    tracker.copy(carrier, CPUStream, CPUStream, key[0], key[1])
    carried, tensors = tracker.deliver([key], CPUStream, CPUStream)
    assert carried == [key] and torch.equal(tensors[0], torch.full((3,), 3.0)) and not tracker.in_transit
    tracker.inbox[key] = tensors[0]
    back = tracker.load(carrier, key[0], key[1])
    back.sum().backward()
    assert torch.equal(src.grad, torch.full((3,), 3.0))
    # a value stashed as None needs no port: it goes straight to the inbox
    tracker.in_transit[key] = None
    assert tracker.deliver([key], CPUStream, CPUStream) == ([], []) and tracker.load(carrier, key[0], key[1]) is None


def _skip_model():
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

    return Stash, Pop


def test_skip_layout_and_verify_skippables():
    Stash, Pop = _skip_model()
    model = nn.Sequential(Stash(), nn.Identity(), Pop())
    verify_skippables(model)
    layout = inspect_skip_layout([nn.Sequential(model[0]), nn.Sequential(model[1]), nn.Sequential(model[2])])
    routes = list(layout.copy_policy(2))
    assert len(routes) == 1 and routes[0][0] == 0 and routes[0][2] == "skip"
    assert layout.requires_copy(routes[0][1], "skip")
    assert list(layout.copy_policy(1)) == []
    with pytest.raises(TypeError):
        verify_skippables(nn.Sequential(Pop()))  # popped but never stashed
    with pytest.raises(TypeError):
        verify_skippables(nn.Sequential(Stash()))  # stashed but never popped
    with pytest.raises(TypeError):
        verify_skippables(nn.Sequential(Stash(), Stash(), Pop(), Pop()))  # same name declared twice without namespaces
    ns1, ns2 = Namespace(), Namespace()
    verify_skippables(nn.Sequential(Stash().isolate(ns1), Stash().isolate(ns2), Pop().isolate(ns2), Pop().isolate(ns1)))


def test_skip_tensors_do_not_leak_after_backward():
    Stash, Pop = _skip_model()
    model = Pipe(nn.Sequential(Stash(), nn.Linear(4, 4), Pop()), balance=[1, 1, 1], devices=["cpu"] * 3, chunks=2, checkpoint="never")
    x = torch.randn(4, 4, requires_grad=True)
    out = model(x)
    ref = weakref.ref(out)
    out.sum().backward()
    del out
    gc.collect()
    assert ref() is None
    assert x.grad is not None
