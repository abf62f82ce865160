import torch
from torch import nn

from fairscale_b200.experimental.tooling.layer_memory_tracker import (
    LayerwiseMemoryTracker,
    find_best_reset_points,
    suggest_checkpoint_location,
)
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP
from fairscale_b200.fair_dev.testing.testing import DummyProcessGroup


def test_reset_points():
    assert find_best_reset_points([1, 1, 1, 1, 1, 1], 2) == (2, [2, 4])
    peak, cuts = find_best_reset_points([10, 1, 1, 1, 12, 2], 2)
    assert peak == 13 and len(cuts) == 2
    assert find_best_reset_points([3, 4], 0) == (7, [])


def test_tracker_records_layers_and_roundtrips(tmp_path):
    model = nn.Sequential(nn.Linear(8, 32), nn.ReLU(), nn.Linear(32, 4))
    tracker = LayerwiseMemoryTracker()
    tracker.monitor(model)
    model(torch.randn(5, 8, requires_grad=True)).sum().backward()
    names = [t.module_name for t in tracker.forward_traces]
    assert names == ["0", "1", "2"]
    assert [t.event.memory_activations for t in tracker.forward_traces] == [5 * 32 * 4, 5 * 32 * 4, 5 * 4 * 4]
    assert tracker.forward_traces[0].module_params == (8 * 32 + 32) * 4
    assert {t.module_name for t in tracker.backward_traces} == {"0", "1", "2"}
    assert tracker.summary.total_activation_allocations == 5 * 68 * 4
    tracker.save_traces(str(tmp_path / "t.json"))
    loaded = LayerwiseMemoryTracker.load(str(tmp_path / "t.json"))
    assert loaded.memory_traces == tracker.memory_traces
    sug = suggest_checkpoint_location(tracker.memory_traces, num_checkpoints=1)
    assert sug.all_modules == names and len(sug.split_modules) == 1
    tracker.stop()
    n = len(tracker.memory_traces)
    model(torch.randn(5, 8)).sum()
    assert len(tracker.memory_traces) == n


def test_tracker_counts_fsdp_all_gathers():
    model = FSDP(nn.Linear(8, 8), process_group=DummyProcessGroup(0, 1))
    tracker = LayerwiseMemoryTracker()
    tracker.monitor(model)
    model(torch.randn(2, 8)).sum().backward()
    tracker.stop()
    assert len(tracker.forward_traces) >= 1


def test_find_best_reset_points_reference_values():
    """Numbers from the reference's tests/experimental/tooling/test_layer_memory_tracker.py:228-254."""
    activations = [10, 8, 8, 9, 7, 7, 5, 4, 4]
    memory, _ = find_best_reset_points(activations, num_checkpoints=0)
    assert memory == sum(activations)
    memory, _ = find_best_reset_points(activations, num_checkpoints=len(activations))
    assert memory == max(activations)
    memory, split_points = find_best_reset_points(activations, num_checkpoints=1)
    assert memory == 35 and split_points == [4]
    memory, split_points = find_best_reset_points(activations, num_checkpoints=2)
    assert memory == 24
    cuts = [0] + split_points + [len(activations)]
    assert max(sum(activations[i:j]) for i, j in zip(cuts[:-1], cuts[1:])) == memory
