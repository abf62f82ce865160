"""Single-process Pipe, case by case on CPU devices (the cases of the reference's tests/nn/pipe/test_pipe.py, test_checkpoint.py,
test_deferred_batch_norm.py, test_microbatch.py, test_balance.py, test_inplace.py, test_bugs.py and skip/test_stash_pop.py,
skip/test_verify_skippables.py, skip/test_gpipe.py that need no GPU): constructor checks and messages, container protocol,
checkpoint modes seen in the autograd graph, inputs of every accepted and refused kind, exceptions and early stop, lock-step
scheduling, deferred batch norm against plain batch norm, micro-batch containers, automatic balancing, skip connections."""
import time
from collections import OrderedDict
from copy import deepcopy

import pytest
import torch
from torch import nn

from fairscale_b200.nn import Pipe
from fairscale_b200.nn.pipe import microbatch
from fairscale_b200.nn.pipe.balance import balance_by_size, balance_by_time, blockpartition
from fairscale_b200.nn.pipe.balance.profile import layerwise_sandbox
from fairscale_b200.nn.pipe.batchnorm import DeferredBatchNorm
from fairscale_b200.nn.pipe.checkpoint import is_checkpointing, is_recomputing
from fairscale_b200.nn.pipe.skip import pop, skippable, stash, verify_skippables
from fairscale_b200.nn.pipe.skip.tracker import SkipTracker, current_skip_tracker, use_skip_tracker

CPU = torch.device("cpu")


def _graph_nodes(grad_fn, seen=None):
    """Class names of every node reachable from ``grad_fn``."""
    seen = set() if seen is None else seen
    if grad_fn is None or grad_fn in seen:
        return []
    seen.add(grad_fn)
    names = [type(grad_fn).__name__]
    for nxt, _ in grad_fn.next_functions:
        names += _graph_nodes(nxt, seen)
    return names


# ------------------------------------------------------------------------------------------------ construction
def test_parameters_and_public_attributes():
    model = nn.Sequential(nn.Linear(1, 1))
    pipe = Pipe(model, balance=[1], devices=["cpu"], chunks=1)
    assert list(pipe.parameters()) != [] and list(pipe.parameters())[0] is model[0].weight
    pipe = Pipe(model, balance=(1,), devices=("cpu",), chunks=42.000, checkpoint=MyString("always"))
    assert isinstance(pipe.balance, list) and isinstance(pipe.devices, list) and isinstance(pipe.chunks, int) and isinstance(pipe.checkpoint, str)
    assert pipe.balance == [1] and pipe.devices == [CPU] and pipe.chunks == 42 and pipe.checkpoint == "always"


class MyString:
    def __init__(self, value):
        self.value = value

    def __str__(self):
        return self.value


@pytest.mark.parametrize("balance", [[2], [1, 1]])
def test_behaves_like_the_sequential_it_wraps(balance):
    a, b = nn.Linear(1, 1), nn.Linear(1, 1)
    pipe = Pipe(nn.Sequential(a, b), balance, devices=["cpu", "cpu"])
    assert len(pipe) == 2 and list(pipe) == [a, b]
    assert pipe[0] is a and pipe[-1] is b and pipe[-2] is a
    for bad in (2, -3):
        with pytest.raises(IndexError):
            pipe[bad]


def test_balance_and_chunks_are_checked():
    two = nn.Sequential(nn.Linear(1, 1), nn.Linear(1, 1))
    with pytest.raises(ValueError, match="different length"):
        Pipe(two, balance=[1])
    with pytest.raises(ValueError, match="different length"):
        Pipe(two, balance=[3])
    with pytest.raises(ValueError, match="positive integer"):
        Pipe(two, balance=[0, 2])
    with pytest.raises(ValueError, match="positive integer"):
        Pipe(two, balance=[-1, 3])
    one = nn.Sequential(nn.Linear(1, 1))
    for chunks in (0, -1):
        with pytest.raises(ValueError, match="chunks must be positive"):
            Pipe(one, balance=[1], devices=["cpu"], chunks=chunks)
    with pytest.raises(ValueError, match="checkpoint is not one of 'always', 'except_last', or 'never'"):
        Pipe(one, balance=[1], devices=["cpu"], chunks=2, checkpoint="INVALID_CHECKPOINT")
    for mode in ("except_last", "always", "never"):  # every mode is fine with a single chunk
        Pipe(one, balance=[1], devices=["cpu"], chunks=1, checkpoint=mode)
    four = nn.Sequential(*[nn.ReLU() for _ in range(4)])
    with pytest.raises(IndexError, match="too few devices"):
        Pipe(four, balance=[1, 1, 1, 1], devices=["cpu"])


def test_messages_point_to_the_balancing_helpers():
    for args in ((nn.Sequential(),), (nn.Sequential(), [1]), (nn.Sequential(nn.Linear(1, 1), nn.Linear(1, 1)), [1])):
        with pytest.raises(ValueError, match=r"nn\.pipe\.balance"):
            Pipe(*args)


def test_module_must_be_a_sequential_without_repeated_children():
    with pytest.raises(TypeError, match="module must be nn.Sequential to be partitioned"):
        Pipe(nn.Module(), [1])
    conv = nn.Conv2d(3, 3, 1)
    with pytest.raises(ValueError, match="module with duplicate children is not supported"):
        Pipe(nn.Sequential(conv, conv), [1, 1])

    class Surrogate(nn.Module):
        def __init__(self, module):
            super().__init__()
            self.module = module

    # the same parameters reachable through two different layers are fine while both sit on one device
    Pipe(nn.Sequential(Surrogate(conv), Surrogate(conv)), [1, 1], devices=["cpu", "cpu"])


def test_extra_devices_are_dropped_partitions_are_module_lists():
    layers = [nn.Linear(1, 1) for _ in range(3)]
    pipe = Pipe(nn.Sequential(*layers), [1, 1, 1], devices=["cpu"] * 5)
    assert pipe.devices == [CPU, CPU, CPU]
    assert isinstance(pipe.partitions, nn.ModuleList) and all(isinstance(p, nn.Sequential) for p in pipe.partitions)
    assert "partitions.0.0.weight" in pipe.state_dict() and "partitions.2.2.bias" in pipe.state_dict()


def test_named_children_keep_their_names_inside_partitions():
    a, b = nn.Linear(1, 1), nn.Linear(1, 1)
    pipe = Pipe(nn.Sequential(OrderedDict([("a", a), ("b", b)])), [1, 1], devices=["cpu", "cpu"])
    names = {n for n, _ in pipe.named_modules()}
    assert {"partitions.0.a", "partitions.1.b"} <= names
    with pytest.raises(AttributeError):
        pipe.a  # unlike nn.Sequential there is no attribute access to the layers


def test_moving_is_denied_casting_is_allowed():
    pipe = Pipe(nn.Sequential(nn.Linear(1, 1), nn.Linear(1, 1)), [1, 1], devices=["cpu", "cpu"])
    for move in (lambda: pipe.cuda(), lambda: pipe.cpu(), lambda: pipe.to(torch.device("cuda")), lambda: pipe.to(0), lambda: pipe.to("cuda"),
                 lambda: pipe.to(device=0), lambda: pipe.to(torch.rand(1)), lambda: pipe.to(tensor=torch.rand(1))):
        with pytest.raises(TypeError, match="denied to move"):
            move()
    pipe.half()
    pipe.to(torch.double)
    pipe.to(dtype=torch.float)
    assert next(pipe.parameters()).dtype == torch.float32


def test_empty_module_passes_tensors_through():
    pipe = Pipe(nn.Sequential(), [])
    assert pipe(torch.tensor(42)) == torch.tensor(42)
    assert pipe((torch.tensor(42),)) == (torch.tensor(42),)
    with pytest.raises(TypeError):
        pipe(42)


# ------------------------------------------------------------------------------------------------ batches
def test_batch_size_that_does_not_divide_or_is_too_small():
    pipe = Pipe(nn.Sequential(nn.Linear(1, 1)), balance=[1], devices=["cpu"], chunks=4)
    for n in (7, 2):  # seven rows in four chunks; two rows give only two micro-batches
        out = pipe(torch.rand(n, 1))
        assert out.shape == (n, 1)
        out.sum().backward()
    # with batch norm a chunk of one row would fail inside the layer, not in the pipe: the pipe does not pad
    small = Pipe(nn.Sequential(nn.Linear(1, 1)), balance=[1], devices=["cpu"], chunks=8)
    assert small(torch.rand(3, 1)).shape == (3, 1)


@pytest.mark.parametrize("mode,checkpointed", [("always", 2), ("except_last", 1), ("never", 0)])
def test_checkpoint_mode_decides_which_micro_batches_recompute(mode, checkpointed):
    pipe = Pipe(nn.Sequential(nn.Linear(1, 1)), balance=[1], devices=["cpu"], chunks=2, checkpoint=mode)
    names = _graph_nodes(pipe(torch.rand(2, 1)).grad_fn)
    assert names.count("CheckpointBackward") == checkpointed
    assert names.count("RecomputeBackward") == checkpointed


def test_eval_mode_has_no_checkpoints():
    pipe = Pipe(nn.Sequential(nn.Linear(1, 1)), balance=[1], devices=["cpu"], chunks=2)
    x = torch.rand(2, 1)
    pipe.train()
    assert {"CheckpointBackward", "RecomputeBackward"} <= set(_graph_nodes(pipe(x).grad_fn))
    pipe.eval()
    assert not {"CheckpointBackward", "RecomputeBackward"} & set(_graph_nodes(pipe(x).grad_fn))


def test_checkpointed_partition_may_pass_a_non_float_tensor():
    class Fork(nn.Module):
        def forward(self, x):
            return x * 2, torch.tensor([False])

    class Join(nn.Module):
        def forward(self, pair):
            return pair[0] * 2

    pipe = Pipe(nn.Sequential(Fork(), Join()), balance=[1, 1], devices=["cpu", "cpu"], chunks=1, checkpoint="always")
    x = torch.rand(1, requires_grad=True)
    pipe(x).backward()
    assert float(x.grad) == 4.0


def test_no_grad_builds_no_graph_inside_the_partitions():
    pipe = Pipe(nn.Sequential(nn.Linear(1, 1)), balance=[1], devices=["cpu"], chunks=2)
    seen = []
    pipe.partitions[0].register_forward_hook(lambda mod, inp, out: seen.append(out))
    with torch.no_grad():
        pipe(torch.rand(2, 1))
    assert seen and all(o.grad_fn is None for o in seen)


def test_inputs_pair_singleton_and_wrong_kinds():
    class Two(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = nn.Linear(1, 1), nn.Linear(1, 1)

        def forward(self, pair):
            return self.a(pair[0]), self.b(pair[1])

    pipe = Pipe(nn.Sequential(Two()), balance=[1], devices=["cpu"], chunks=2)
    a, b = torch.rand(10, 1, requires_grad=True), torch.rand(10, 1, requires_grad=True)
    out_a, out_b = pipe((a, b))
    (out_a + out_b).mean().backward()
    assert a.grad is not None and b.grad is not None

    class One(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = nn.Linear(1, 1)

        def forward(self, only):
            return (self.fc(only[0]),)

    pipe = Pipe(nn.Sequential(One()), balance=[1], devices=["cpu"], chunks=2)
    a = torch.rand(10, 1, requires_grad=True)
    (out,) = pipe((a,))
    out.mean().backward()
    assert a.grad is not None and all(p.grad is not None for p in pipe.parameters())

    pipe = Pipe(nn.Sequential(nn.Linear(1, 1)), balance=[1], devices=["cpu"])
    with pytest.raises(TypeError):
        pipe(torch.rand(1), torch.rand(1))  # one positional input only
    with pytest.raises(TypeError):
        pipe("hello")
    with pytest.raises(TypeError):
        pipe((torch.rand(1), "hello"))


def test_layers_must_return_tensors():
    class Word(nn.Module):
        def forward(self, _):
            return "hello"

    class TensorAndWord(nn.Module):
        def forward(self, x):
            return x, "hello"

    for layer in (Word(), TensorAndWord()):
        with pytest.raises(TypeError):
            Pipe(nn.Sequential(layer), balance=[1], devices=["cpu"])(torch.rand(1))


# ------------------------------------------------------------------------------------------------ scheduling and failures
def test_exception_of_a_layer_reaches_the_caller_and_stops_the_earlier_stages():
    class Expected(Exception):
        pass

    class Raise(nn.Module):
        def forward(self, *_):
            raise Expected()

    with pytest.raises(Expected):
        Pipe(nn.Sequential(Raise()), balance=[1], devices=["cpu"], chunks=1)(torch.rand(1))

    counted = []

    class Count(nn.Module):
        def forward(self, x):
            time.sleep(0.1)
            counted.append(1)
            return x

    model = nn.Sequential(nn.Identity(), nn.ReLU(), Count(), Raise())
    pipe = Pipe(model, [1, 1, 1, 1], devices=["cpu"] * 4, chunks=3)
    with pytest.raises(Expected):
        pipe(torch.rand(3))
    assert len(counted) == 2  # the third micro-batch never entered the stage before the failing one


def test_stages_advance_in_lock_step():
    timeline = []

    class Log(nn.Module):
        def __init__(self, stage, seconds):
            super().__init__()
            self.stage, self.seconds, self.count = stage, seconds, 0

        def forward(self, x):
            time.sleep(self.seconds)
            timeline.append((self.count, self.stage))
            self.count += 1
            return x

    pipe = Pipe(nn.Sequential(Log(0, 0.0), Log(1, 0.1)), balance=[1, 1], devices=["cpu", "cpu"], chunks=3)
    pipe(torch.rand(3, 1))
    # stage 0 does not run ahead of the clock: micro-batch 2 enters it only when stage 1 takes micro-batch 1
    assert timeline == [(0, 0), (1, 0), (0, 1), (2, 0), (1, 1), (2, 1)]


def test_user_autograd_functions_and_thread_local_state():
    """A custom Function's backward runs in the thread of the stage that ran its forward... whichever thread it is, the
    result must be that of the plain module."""
    class Double(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            return x * 2

        @staticmethod
        def backward(ctx, g):
            return g * 2

    class Layer(nn.Module):
        def forward(self, x):
            return Double.apply(x)

    pipe = Pipe(nn.Sequential(Layer(), Layer()), [1, 1], devices=["cpu", "cpu"], chunks=2, checkpoint="always")
    x = torch.rand(4, 1, requires_grad=True)
    pipe(x).sum().backward()
    assert torch.equal(x.grad, torch.full_like(x, 4.0))


def test_random_layers_draw_the_same_numbers_when_recomputed():
    class Drop(nn.Module):
        def forward(self, x):
            return nn.functional.dropout(x, p=0.5, training=True)

    x = torch.ones(8, 64, requires_grad=True)
    pipe = Pipe(nn.Sequential(Drop(), Drop()), [1, 1], devices=["cpu", "cpu"], chunks=4, checkpoint="always")
    out = pipe(x)
    out.sum().backward()
    # d out / d x is the mask product (times 4): it matches the forward's mask only if the recomputation replayed it
    assert torch.equal(x.grad != 0, out.detach() != 0)


def test_inplace_operations():
    # nothing requires grad: an in-place layer on the (detached) micro-batches is fine
    pipe = Pipe(nn.Sequential(nn.Identity(), nn.ReLU(inplace=True)), [1, 1], devices=["cpu", "cpu"], checkpoint="never")
    x = torch.rand(3) - 0.5
    assert torch.equal(pipe(x.clone()), x.clamp(min=0))
    # in place on a leaf that requires grad is reported, by the forward or by the backward
    leaf = torch.rand(1, requires_grad=True)
    with pytest.raises(RuntimeError, match="[Ii]n-?place"):
        Pipe(nn.Sequential(nn.ReLU(inplace=True)), [1], devices=["cpu"], checkpoint="always")(leaf).backward()


def test_checkpoints_are_recomputed_in_reverse_order_and_flags_are_visible():
    order, flags = [], []

    class Log(torch.autograd.Function):
        @staticmethod
        def forward(ctx, name, x):
            ctx.name = name
            return x.detach()

        @staticmethod
        def backward(ctx, g):
            order.append(ctx.name)
            return None, g

    class Probe(nn.Module):
        def __init__(self, name):
            super().__init__()
            self.name = name

        def forward(self, x):
            flags.append((self.name, is_checkpointing(), is_recomputing()))
            return Log.apply(self.name, x)

    pipe = Pipe(nn.Sequential(Probe("a"), Probe("b")), [1, 1], devices=["cpu", "cpu"], chunks=1, checkpoint="always")
    x = torch.rand(2, requires_grad=True)
    pipe(x).sum().backward()
    assert order == ["b", "a"]
    assert flags[:2] == [("a", True, False), ("b", True, False)]          # forward: under a checkpoint
    assert sorted(flags[2:]) == [("a", False, True), ("b", False, True)]   # backward: being recomputed
    flags.clear()
    Pipe(nn.Sequential(Probe("c")), [1], devices=["cpu"], chunks=1, checkpoint="never")(x)
    assert flags == [("c", False, False)]


def test_inputs_that_need_no_gradient():
    pipe = Pipe(nn.Sequential(nn.Linear(1, 1)), balance=[1], devices=["cpu"], chunks=2, checkpoint="always")
    out = pipe(torch.rand(2, 1))  # the parameters still do
    out.sum().backward()
    assert pipe[0].weight.grad is not None

    class Const(nn.Module):
        def forward(self, x):
            return x.detach() * 2

    x = torch.rand(2, 1, requires_grad=True)
    assert not Pipe(nn.Sequential(Const()), [1], devices=["cpu"], chunks=2, checkpoint="never")(x).requires_grad
    # a checkpointed micro-batch always carries a graph (its recomputation hangs on it), whatever the layer returned
    out = Pipe(nn.Sequential(Const()), [1], devices=["cpu"], chunks=2, checkpoint="always")(x)
    out.sum().backward()
    assert x.grad is None or float(x.grad.abs().sum()) == 0.0


# ------------------------------------------------------------------------------------------------ deferred batch norm
@pytest.mark.parametrize("mode", ["never", "always", "except_last"])
def test_deferred_batch_norm_tracks_the_mini_batch_statistics(mode):
    torch.manual_seed(0)
    bn = nn.BatchNorm2d(3)
    pipe = Pipe(nn.Sequential(deepcopy(bn)), balance=[1], devices=["cpu"], chunks=2, checkpoint=mode, deferred_batch_norm=True)
    x = torch.rand(4, 3, 10, 10)
    pipe(x).mean().backward()
    bn(x).mean().backward()
    assert isinstance(pipe[0], DeferredBatchNorm)
    torch.testing.assert_close(pipe[0].running_mean, bn.running_mean, atol=1e-4, rtol=0)
    torch.testing.assert_close(pipe[0].running_var, bn.running_var, atol=1e-4, rtol=0)


@pytest.mark.parametrize("mode", ["never", "always"])
def test_deferred_batch_norm_gradients_with_one_chunk(mode):
    torch.manual_seed(0)
    bn = nn.BatchNorm2d(3)
    pipe = Pipe(nn.Sequential(deepcopy(bn)), balance=[1], devices=["cpu"], chunks=1, checkpoint=mode, deferred_batch_norm=True)
    x = torch.rand(4, 3, 10, 10)
    pipe(x).mean().backward()
    bn(x).mean().backward()
    torch.testing.assert_close(pipe[0].weight.grad, bn.weight.grad, atol=1e-4, rtol=0)
    torch.testing.assert_close(pipe[0].bias.grad, bn.bias.grad, atol=1e-4, rtol=0)


@pytest.mark.parametrize("momentum", [0.1, None])
def test_deferred_batch_norm_layer_alone(momentum):
    torch.manual_seed(0)
    chunks = 4
    bn = nn.BatchNorm2d(3, momentum=momentum)
    dbn = DeferredBatchNorm.convert_deferred_batch_norm(deepcopy(bn), chunks=chunks)
    assert isinstance(dbn, DeferredBatchNorm) and DeferredBatchNorm.convert_deferred_batch_norm(dbn, chunks) is dbn
    for step in range(3):
        x = torch.rand(8, 3, 6, 6) + step
        bn(x)
        for piece in x.chunk(chunks):
            dbn(piece)
        torch.testing.assert_close(dbn.running_mean, bn.running_mean, atol=1e-4, rtol=0)
        torch.testing.assert_close(dbn.running_var, bn.running_var, atol=1e-3, rtol=0)
    assert int(dbn.num_batches_tracked) == 3
    # eval: the running statistics are used and left alone
    dbn.eval()
    bn.eval()
    before = dbn.running_mean.clone()
    x = torch.rand(8, 3, 6, 6)
    # running variances differ by the factor n / (n - 1): batch norm keeps the unbiased estimate, the deferred layer the biased one
    torch.testing.assert_close(dbn(x), bn(x), atol=2e-2, rtol=1e-2)
    assert torch.equal(dbn.running_mean, before)


def test_deferred_batch_norm_in_a_training_loop_with_conv():
    torch.manual_seed(0)
    plain = nn.Sequential(nn.Conv2d(3, 3, 1), nn.BatchNorm2d(3))
    pipe = Pipe(deepcopy(plain), [1, 1], devices=["cpu", "cpu"], chunks=2, deferred_batch_norm=True)
    opts = [torch.optim.SGD(m.parameters(), lr=0.1) for m in (plain, pipe)]
    for step in range(3):
        x = torch.rand(6, 3, 4, 4)
        for m, o in zip((plain, pipe), opts):
            o.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    # normalisation inside a micro-batch uses that micro-batch's statistics, so outputs differ a little; the running
    # statistics (what evaluation uses) follow the mini-batch and stay close
    torch.testing.assert_close(pipe[1].running_mean, plain[1].running_mean, atol=5e-2, rtol=0)
    x = torch.rand(4, 3, 4, 4, requires_grad=True)
    pipe(x).mean().backward()
    assert x.grad is not None


# ------------------------------------------------------------------------------------------------ micro-batches
def test_batch_container():
    x = torch.tensor(42.0)
    single = microbatch.Batch(x, 0)
    assert single.atomic and single.tensor is x and single.tensor_or_tensors is x and single.index == 0
    with pytest.raises(AttributeError):
        single.tensors
    assert list(single) == [x] and len(single) == 1 and single[0] is x
    pair = microbatch.Batch((x, x + 1), 3)
    assert not pair.atomic and pair.tensors == (x, x + 1) and pair.index == 3 and len(pair) == 2
    with pytest.raises(AttributeError):
        pair.tensor
    assert pair[1] is pair.tensors[1] and list(pair)[0] is x

    doubled = single.call(lambda t: t * 2)
    assert float(doubled.tensor) == 84.0 and doubled.index == 0
    swapped = pair.call(lambda ts: (ts[1], ts[0]))
    assert float(swapped[0]) == 43.0

    single[0] = x + 5
    assert float(single.tensor) == 47.0
    single[:] = (x,)
    assert single.tensor is x
    pair[0] = x + 9
    assert float(pair[0]) == 51.0
    pair[:] = (x, x)
    assert pair.tensors == (x, x)


def test_check_scatter_gather():
    microbatch.check(torch.tensor(1))
    microbatch.check((torch.tensor(1), torch.tensor(2)))
    for bad in (42, "x", (torch.tensor(1), 2), [torch.tensor(1)]):
        with pytest.raises(TypeError):
            microbatch.check(bad)

    x = torch.arange(12.0).view(6, 2)
    parts = microbatch.scatter(x, chunks=3)
    assert [p.tensor.shape[0] for p in parts] == [2, 2, 2] and [p.index for p in parts] == [0, 1, 2]
    assert torch.equal(microbatch.gather(parts), x)
    a, b = microbatch.scatter((x, x + 100), chunks=2)
    assert a.tensors[1].shape == (3, 2) and float(b.tensors[1][0, 0]) == 106.0
    whole = microbatch.gather([a, b])
    assert isinstance(whole, tuple) and torch.equal(whole[0], x) and torch.equal(whole[1], x + 100)
    assert len(microbatch.scatter(torch.zeros(2, 1), chunks=8)) == 2  # never more micro-batches than rows


# ------------------------------------------------------------------------------------------------ balancing
def test_block_partition():
    assert blockpartition.solve([1, 2, 3, 4, 5, 6], partitions=2) == [[1, 2, 3, 4], [5, 6]]
    assert blockpartition.solve([0, 0], partitions=2) == [[0], [0]]
    with pytest.raises(ValueError):
        blockpartition.solve([42], partitions=0)
    with pytest.raises(ValueError):
        blockpartition.solve([42], partitions=-1)
    with pytest.raises(ValueError):
        blockpartition.solve([], partitions=1)
    with pytest.raises(ValueError):
        blockpartition.solve([42], partitions=2)  # fewer items than partitions


def test_balance_by_time_follows_the_slow_layers():
    class Delay(nn.Module):
        def __init__(self, seconds):
            super().__init__()
            self.seconds = seconds

        def forward(self, x):
            time.sleep(self.seconds)
            return x

    model = nn.Sequential(*[Delay(i / 100) for i in [1, 2, 3, 4, 5, 6]])
    assert balance_by_time(2, model, torch.rand(1), device="cpu", timeout=0.5) == [4, 2]
    # profiling works on copies: the module's mode and parameters are not touched
    model = nn.Sequential(nn.Linear(2, 2), nn.Dropout(), nn.Linear(2, 2))
    model.eval()
    before = deepcopy(model.state_dict())
    balance_by_time(1, model, torch.rand(1, 2), device="cpu", timeout=0.05)
    assert not model.training and all(torch.equal(v, before[k]) for k, v in model.state_dict().items())
    # tuples flow through
    class Twin(nn.Module):
        def forward(self, pair):
            return pair[0] + 1, pair[1] + 1

    assert sum(balance_by_time(2, nn.Sequential(Twin(), Twin(), Twin()), (torch.rand(1), torch.rand(1)), device="cpu", timeout=0.05)) == 3


def test_balance_by_size_needs_a_device_that_reports_memory():
    model = nn.Sequential(*[nn.Linear(10, 10) for _ in range(4)])
    with pytest.raises(ValueError, match="size profiler supports only CUDA device"):
        balance_by_size(2, model, torch.rand(4, 10), device="cpu")


def test_profiling_sandbox_yields_copies_in_training_mode():
    model = nn.Sequential(nn.BatchNorm1d(3), nn.Linear(3, 3))
    model.eval()
    for original, layer in zip(model, layerwise_sandbox(model, CPU)):
        assert layer is not original and layer.training and not original.training
        assert all(p.device == CPU for p in layer.parameters())
        for p in layer.parameters():
            p.data.zero_()
    assert float(model[1].weight.abs().sum()) > 0.0  # the originals were not written


# ------------------------------------------------------------------------------------------------ skip connections
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


@pytest.mark.parametrize("balance", [[3], [1, 2], [2, 1], [1, 1, 1]])
@pytest.mark.parametrize("mode", ["never", "always", "except_last"])
def test_skip_connection_over_any_partitioning(balance, mode):
    model = nn.Sequential(Stash(), nn.Linear(4, 4), Pop())
    pipe = Pipe(deepcopy(model), balance, devices=["cpu"] * len(balance), chunks=3, checkpoint=mode)
    x = torch.rand(6, 4, requires_grad=True)
    x2 = x.detach().clone().requires_grad_()
    out = pipe(x)
    want = model[1](x2 * 2) + x2
    torch.testing.assert_close(out, want)
    out.sum().backward()
    want.sum().backward()
    torch.testing.assert_close(x.grad, x2.grad)
    torch.testing.assert_close(pipe[1].weight.grad, model[1].weight.grad)


def test_skip_of_none_and_layers_without_skips():
    @skippable(stash=["none"])
    class StashNone(nn.Module):
        def forward(self, x):
            yield stash("none", None)
            return x

    @skippable(pop=["none"])
    class PopNone(nn.Module):
        def forward(self, x):
            nothing = yield pop("none")
            assert nothing is None
            return x + 1

    pipe = Pipe(nn.Sequential(StashNone(), PopNone()), [1, 1], devices=["cpu", "cpu"], chunks=2)
    assert torch.equal(pipe(torch.zeros(4, 1)), torch.ones(4, 1))

    @skippable()
    class Plain(nn.Module):
        def forward(self, x):
            return x * 3

    assert float(Plain()(torch.ones(1))) == 3.0  # a skippable without declarations is an ordinary module


def test_stash_and_pop_must_match_their_declarations():
    @skippable(stash=["declared"])
    class StashesOther(nn.Module):
        def forward(self, x):
            yield stash("other", x)
            return x

    @skippable(pop=["declared"])
    class PopsOther(nn.Module):
        def forward(self, x):
            y = yield pop("other")
            return x + y

    @skippable(stash=["declared"])
    class Forgets(nn.Module):
        def forward(self, x):
            return x

    with pytest.raises(RuntimeError, match="'other' has not been declared as stashable"):
        StashesOther()(torch.rand(1))
    with pytest.raises(RuntimeError, match="must be stashed but have not"):
        Forgets()(torch.rand(1))
    # popping what nobody stashed, under a name that is declared and under one that is not
    with use_skip_tracker(SkipTracker()):
        with pytest.raises(RuntimeError, match="'skip' has not been stashed"):
            Pop()(torch.rand(1))
        with pytest.raises(RuntimeError, match="has not been stashed|'other' has not been declared as poppable"):
            PopsOther()(torch.rand(1))
    # outside a pipe the default tracker carries the tensor from one call to the next
    s, p = Stash(), Pop()
    x = torch.rand(2)
    assert torch.equal(p(s(x)), x * 3)
    assert isinstance(current_skip_tracker(), SkipTracker)
    mine = SkipTracker()
    with use_skip_tracker(mine):
        assert current_skip_tracker() is mine
    assert current_skip_tracker() is not mine


def test_skippables_are_verified_before_anything_runs():
    verify_skippables(nn.Sequential(Stash(), Pop()))
    with pytest.raises(TypeError, match="declared 'skip' as poppable but it was not stashed"):
        verify_skippables(nn.Sequential(Pop()))
    with pytest.raises(TypeError, match="no module declared 'skip' as poppable but stashed"):
        verify_skippables(nn.Sequential(Stash()))
    with pytest.raises(TypeError, match="redeclared 'skip' as stashable but not isolated by namespace"):
        verify_skippables(nn.Sequential(Stash(), Stash(), Pop()))
    with pytest.raises(TypeError, match="redeclared 'skip' as poppable but not isolated by namespace"):
        verify_skippables(nn.Sequential(Stash(), Pop(), Pop()))

    @skippable(stash=["both"], pop=["both"])
    class Both(nn.Module):
        def forward(self, x):
            return x

    with pytest.raises(TypeError, match="declared 'both' both as stashable and as poppable"):
        verify_skippables(nn.Sequential(Both()))
    with pytest.raises(TypeError):
        Pipe(nn.Sequential(Stash()), [1], devices=["cpu"])
    # the same name in two isolated namespaces is two different skips
    from fairscale_b200.nn.pipe.skip import Namespace

    ns1, ns2 = Namespace(), Namespace()
    verify_skippables(nn.Sequential(Stash().isolate(ns1), Pop().isolate(ns1), Stash().isolate(ns2), Pop().isolate(ns2)))
    model = nn.Sequential(Stash().isolate(ns1), Stash().isolate(ns2), Pop().isolate(ns2), Pop().isolate(ns1))
    pipe = Pipe(model, [2, 2], devices=["cpu", "cpu"], chunks=2)
    x = torch.rand(4, 2)
    torch.testing.assert_close(pipe(x), (x * 4 + x * 2) + x)
    assert "Stash" in repr(Stash())


@pytest.mark.parametrize("mode", ["always", "except_last"])
def test_recomputation_runs_under_the_autocast_state_of_the_forward(mode):
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(4, 8), nn.Tanh(), nn.Linear(8, 8), nn.Tanh(), nn.Linear(8, 2))
    plain = deepcopy(model)
    pipe = Pipe(model, [2, 2, 1], devices=["cpu"] * 3, chunks=2, checkpoint=mode)
    x = torch.randn(4, 4, requires_grad=True)
    x2 = x.detach().clone().requires_grad_()
    with torch.autocast("cpu", dtype=torch.bfloat16):
        out, want = pipe(x), plain(x2)
    assert out.dtype == torch.bfloat16
    out.float().sum().backward()  # backward starts with autocast off; the stages got bf16 activations from their predecessors
    want.float().sum().backward()
    torch.testing.assert_close(x.grad, x2.grad, atol=2e-2, rtol=2e-2)
    for a, b in zip(pipe.parameters(), plain.parameters()):
        torch.testing.assert_close(a.grad, b.grad, atol=2e-2, rtol=2e-2)
