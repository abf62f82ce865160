"""The test-support package users of the reference import in their own test suites (``fairscale.fair_dev.testing``):
deep comparison of nested containers, model comparison helpers (local and across ranks), temporary files, the GPT-2
stand-in model, the device / dtype checking module, world-size helpers and the memory probes."""
import os

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing import testing as T
from fairscale_b200.fair_dev.testing.testing_memory import find_tensor_by_shape


def test_objects_are_equal_on_nested_containers():
    a = {"w": torch.ones(2, 2), "nested": [torch.zeros(3), (1, "x", torch.arange(3))], "n": 5}
    b = {"w": torch.ones(2, 2), "nested": [torch.zeros(3), (1, "x", torch.arange(3))], "n": 5}
    assert T.objects_are_equal(a, b)
    b["nested"][1] = (1, "x", torch.arange(3) + 1)
    assert not T.objects_are_equal(a, b)
    with pytest.raises((ValueError, AssertionError)):
        T.objects_are_equal(a, b, raise_exception=True)
    assert not T.objects_are_equal([1, 2], (1, 2))                      # the container type counts
    assert not T.objects_are_equal({"a": 1}, {"b": 1}) and not T.objects_are_equal([1], [1, 2])
    with pytest.raises(ValueError, match="dict key 'w'"):
        T.objects_are_equal({"w": torch.ones(2)}, {"w": torch.zeros(2)}, raise_exception=True)
    # tolerances reach the leaves
    assert T.objects_are_equal([torch.ones(2)], [torch.ones(2) + 1e-3], rtol=1e-2, atol=1e-2)
    assert not T.objects_are_equal([torch.ones(2)], [torch.ones(2) + 1e-3], rtol=1e-6, atol=1e-6)


def test_model_comparison_and_norm_helpers():
    torch.manual_seed(0)
    m1, m2 = nn.Linear(3, 3), nn.Linear(3, 3)
    with pytest.raises(AssertionError, match="parameters differ"):
        T.check_same_model_params(m1, m2, "after init")
    m2.load_state_dict(m1.state_dict())
    T.check_same_model_params(m1, m2)
    sd = {"a": torch.full((4,), 3.0), "idx": torch.arange(4)}   # integer entries are skipped
    torch.testing.assert_close(T.state_dict_norm(sd), torch.tensor([6.0]))


def test_temporary_files_and_directories():
    with T.temp_files_ctx(3) as files:
        assert len(files) == 3 and all(os.path.exists(f) for f in files)
        T.rmf(files[0])
        T.rmf(files[0])  # removing twice is fine
    assert not any(os.path.exists(f) for f in files)
    here = os.getcwd()
    with T.in_temporary_directory() as d:
        assert os.path.realpath(os.getcwd()) == os.path.realpath(d)
    assert os.getcwd() == here and not os.path.exists(d)


def test_stand_in_models_and_modules():
    torch.manual_seed(1)
    gpt = T.GPT2(embed_dim=16, num_heads=2, num_layers=2, num_positions=12, num_vocab=20, num_classes=4)
    tokens = torch.randint(0, 20, (12, 3))  # [batch, sequence]
    assert gpt(tokens).shape == (3, 12, 20)  # language-model logits, sequence first
    out = gpt(tokens, classify=True)
    outs = out if isinstance(out, (tuple, list)) else (out,)
    assert all(torch.isfinite(o).all() for o in outs) and {o.shape[-1] for o in outs} <= {20, 4}
    sum(o.sum() for o in outs).backward()
    assert all(p.grad is not None for p in gpt.parameters())

    check = T.DeviceAndTypeCheckModule(expected_input_dtype=torch.float32, expected_input_device=torch.device("cpu"),
                                       expected_param_dtype=torch.float32, expected_loss_dtype=torch.float32)
    loss = check(torch.randn(2, 5))
    assert loss.dim() == 0
    with pytest.raises(AssertionError):
        check(torch.randn(2, 5).double())

    ident = T.IdentityLayer((2, 3), scale=0.5)
    assert ident().shape == (2, 3) and ident.weight.requires_grad

    group = T.DummyProcessGroup(rank=1, size=4)
    assert group.rank() == 1 and group.size() == 4


def test_world_size_helpers_and_environment_probes():
    sizes = T.get_world_sizes()
    assert sizes and all(isinstance(s, int) and s >= 1 for s in sizes)
    assert isinstance(T.in_circle_ci(), bool)
    assert isinstance(T.torch_cuda_version(), tuple)
    assert T.get_smi_memory() >= 0.0
    port = T.find_free_port()
    assert 1024 < port < 65536


def _across_ranks(rank, world):
    torch.manual_seed(0)
    same = nn.Sequential(nn.Linear(3, 3), nn.BatchNorm1d(3))
    T.check_same_models_across_ranks(same, dist.group.WORLD, params_should_be_equal=True, check_broadcast_buffers=True)
    torch.manual_seed(rank)
    different = nn.Linear(3, 3, bias=False)  # one parameter: the failing comparison below ends after one collective
    T.check_same_models_across_ranks(different, dist.group.WORLD, params_should_be_equal=False, check_broadcast_buffers=False)
    if rank == 0:
        with pytest.raises(AssertionError):
            T.check_same_models_across_ranks(different, dist.group.WORLD, params_should_be_equal=True, check_broadcast_buffers=False)
    else:
        T.check_same_models_across_ranks(different, dist.group.WORLD, params_should_be_equal=True, check_broadcast_buffers=False)


def test_models_are_compared_across_ranks():
    T.spawn_ranks(_across_ranks, 2, (), backend="gloo")


def test_find_tensor_by_shape_sees_live_parameters_only():
    keep = nn.Parameter(torch.zeros(7, 13))
    assert find_tensor_by_shape((7, 13))
    assert not find_tensor_by_shape((7, 14))
    plain = torch.zeros(5, 17)
    assert not find_tensor_by_shape((5, 17)) and find_tensor_by_shape((5, 17), only_param=False)
    del keep, plain
