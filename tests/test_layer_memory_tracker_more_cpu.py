"""LayerwiseMemoryTracker beyond the basics (cases of the reference's tests/experimental/tooling/test_layer_memory_tracker.py
in a form that needs no GPU: activation sizes are counted from the tensors, allocator figures are zero on CPU): nested models
record their leaves in execution order, views are not counted as activations, the largest producers, the summary, clearing and
restarting, suggested checkpoint places with skipped layers, all-gather volumes of FSDP on two ranks (per layer and
cumulative, only for the tracked process group), serialisation of both event kinds, and the plotting entry point."""
import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.experimental.tooling.layer_memory_tracker import (
    LayerMemoryTrace,
    LayerwiseMemoryTracker,
    ProcessGroupTracker,
    TraceBackwardEvent,
    TraceForwardEvent,
    compare_memory_traces_in_plot,
    find_best_reset_points,
    null_context,
    suggest_checkpoint_location,
)
from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP


class _Block(nn.Module):
    def __init__(self, width):
        super().__init__()
        self.fc = nn.Linear(width, width)
        self.act = nn.ReLU()

    def forward(self, x):
        return self.act(self.fc(x))


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.stem = nn.Linear(4, 16)
        self.blocks = nn.Sequential(_Block(16), _Block(16))
        self.flat = nn.Flatten()  # a view: allocates nothing
        self.head = nn.Linear(16, 2)

    def forward(self, x):
        return self.head(self.flat(self.blocks(self.stem(x))))


def test_nested_model_records_leaves_in_execution_order():
    torch.manual_seed(0)
    model, tracker = _Net(), LayerwiseMemoryTracker()
    tracker.monitor(model)
    x = torch.randn(3, 4, requires_grad=True)
    model(x).sum().backward()
    fwd = tracker.forward_traces
    assert [t.module_name for t in fwd] == ["stem", "blocks.0.fc", "blocks.0.act", "blocks.1.fc", "blocks.1.act", "flat", "head"]
    row = 3 * 16 * 4
    assert [t.event.memory_activations for t in fwd] == [row, row, row, row, row, 0, 3 * 2 * 4]
    assert [t.module_params for t in fwd] == [(4 * 16 + 16) * 4, (16 * 16 + 16) * 4, 0, (16 * 16 + 16) * 4, 0, 0, (16 * 2 + 2) * 4]
    assert all(t.allocated == 0 and t.reserved == 0 and t.event.memory_diff == 0 for t in fwd) or torch.cuda.is_available()
    # backward comes in reverse order, for the same leaves
    bwd = [t.module_name for t in tracker.backward_traces]
    assert bwd[0] == "head" and set(bwd) <= {t.module_name for t in fwd} and "stem" in bwd
    assert all(isinstance(t.event, TraceBackwardEvent) for t in tracker.backward_traces)
    assert len(tracker.memory_traces) == len(fwd) + len(bwd)

    top = tracker.top_forward_activation_producers(top=3)
    assert len(top) == 3 and all(t.event.memory_activations == row for t in top)
    summary = tracker.summary
    assert summary.total_activation_allocations == 5 * row + 3 * 2 * 4
    assert summary.top_forward_activation_producers[0].event.memory_activations == row
    assert summary.max_memory_allocated == tracker.max_memory_allocated and summary.max_memory_cached == tracker.max_memory_cached

    # clearing keeps the hooks: the next pass is recorded afresh; stopping removes them
    tracker.clear_traces()
    assert tracker.memory_traces == []
    with torch.no_grad():
        model(x)
    assert len(tracker.forward_traces) == 7 and tracker.backward_traces == []
    tracker.stop()
    tracker.clear_traces()
    model(x)
    assert tracker.memory_traces == []
    tracker.stop()  # twice is harmless


def test_suggested_checkpoints_and_skipped_layers():
    def trace(name, size, forward=True):
        event = TraceForwardEvent(memory_diff=size, memory_activations=size) if forward else TraceBackwardEvent(memory_activations=size)
        return LayerMemoryTrace(module_name=name, module_params=0, allocated=0, reserved=0, is_forward=forward, all_gathered=0,
                                cumul_all_gathered=0, event=event)

    sizes = [10, 8, 8, 9, 7, 7, 5, 4, 4]
    traces = [trace(f"layer{i}", s) for i, s in enumerate(sizes)] + [trace(f"layer{i}", 1, forward=False) for i in range(9)]
    none = suggest_checkpoint_location(traces, num_checkpoints=0)
    assert none.max_memory == sum(sizes) and none.split_modules == [] and none.all_modules == [f"layer{i}" for i in range(9)]
    one = suggest_checkpoint_location(traces, num_checkpoints=1)
    assert one.max_memory == 35 and one.split_modules == ["layer4"]
    two = suggest_checkpoint_location(traces, num_checkpoints=2)
    assert two.max_memory == 24 and len(two.split_modules) == 2
    # the first layers (an embedding, say) can be left out of the search
    skipped = suggest_checkpoint_location(traces, num_checkpoints=1, num_skipped_layers=2)
    assert skipped.all_modules[0] == "layer2" and skipped.max_memory == find_best_reset_points(sizes[2:], 1)[0]
    # a module that runs twice is listed once
    twice = suggest_checkpoint_location(traces[:3] + traces[:3], num_checkpoints=1)
    assert twice.all_modules == ["layer0", "layer1", "layer2"]


def test_reset_points_are_optimal_on_small_inputs():
    import itertools

    for sizes in ([5, 1, 1, 5], [1, 2, 3, 4, 5], [7], [3, 3, 3, 3, 3, 3]):
        for k in range(0, len(sizes) + 1):
            peak, cuts = find_best_reset_points(sizes, k)
            assert cuts == sorted(cuts) and len(cuts) <= max(k, 0)
            best = min(
                max(sum(sizes[a:b]) for a, b in zip((0,) + c, c + (len(sizes),)))
                for n in range(0, min(k, len(sizes) - 1) + 1) for c in itertools.combinations(range(1, len(sizes)), n)
            )
            assert peak == best, (sizes, k, peak, best)


def test_traces_round_trip_through_dicts_and_files(tmp_path):
    fwd = LayerMemoryTrace("a.b", 12, 100, 200, True, 7, 9, TraceForwardEvent(memory_diff=3, memory_activations=5))
    bwd = LayerMemoryTrace("a.b", 12, 90, 200, False, 0, 0, TraceBackwardEvent(memory_activations=4))
    for t in (fwd, bwd):
        again = LayerMemoryTrace.from_dict(t.to_dict())
        assert again == t and type(again.event) is type(t.event)
    tracker = LayerwiseMemoryTracker()
    tracker.memory_traces = [fwd, bwd]
    tracker.save_traces(str(tmp_path / "traces.json"))
    loaded = LayerwiseMemoryTracker.load(str(tmp_path / "traces.json"))
    assert loaded.memory_traces == [fwd, bwd] and loaded.max_memory_allocated == 100 and loaded.max_memory_cached == 200
    with null_context():
        pass


def test_plotting_needs_matplotlib_and_says_so():
    try:
        import matplotlib  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="matplotlib"):
            compare_memory_traces_in_plot({"run": []})
        with pytest.raises(ImportError, match="matplotlib"):
            LayerwiseMemoryTracker().show_plots(capture=True)
    else:
        png = compare_memory_traces_in_plot({"run": []}, capture=True)
        assert png[:4] == b"\x89PNG"


# ------------------------------------------------------------------------------------------------ all-gathers of FSDP
def _fsdp_all_gathers(rank, world, track_group):
    torch.manual_seed(0)
    group = dist.new_group(list(range(world)))
    other = dist.new_group(list(range(world)))
    model = nn.Sequential(nn.Linear(8, 8, bias=False), nn.Linear(8, 8, bias=False), nn.Linear(8, 4, bias=False))
    wrapped_group = ProcessGroupTracker(group) if track_group else group
    inner = [FSDP(layer, process_group=wrapped_group, flatten_parameters=True) for layer in model]
    fsdp = FSDP(nn.Sequential(*inner), process_group=wrapped_group)
    tracker = LayerwiseMemoryTracker()
    tracker.monitor(fsdp)
    fsdp(torch.randn(2, 8)).sum().backward()
    dist.all_gather([torch.empty(4) for _ in range(world)], torch.ones(4), group=other)  # somebody else's traffic
    tracker.stop()
    fwd = tracker.forward_traces
    assert len(fwd) == 3
    # each wrapped layer gathered its own weight (fp32) before it ran: 8*8, 8*8, 4*8 elements
    assert [t.all_gathered for t in fwd] == [8 * 8 * 4, 8 * 8 * 4, 4 * 8 * 4], [t.all_gathered for t in fwd]
    # cumulative: what the FSDP instances around the layer hold gathered while it runs; every wrapped layer here frees its
    # weight after its forward and the outer instance has no parameters of its own, so it is the layer's own gather
    assert [t.cumul_all_gathered for t in fwd] == [t.all_gathered for t in fwd]
    # backward gathers again (the shards were freed after forward)
    assert sum(t.all_gathered for t in tracker.backward_traces) > 0


@pytest.mark.parametrize("track_group", [True, False])
def test_fsdp_all_gather_volumes_per_layer(track_group):
    spawn_ranks(_fsdp_all_gathers, 2, (track_group,), backend="gloo")
