"""Sharded checkpoints of FSDP put together without the model (cases of the reference's
tests/nn/data_parallel/test_fsdp_metadata.py on gloo ranks): every rank saves ``local_state_dict()`` and
``local_metadata_dict()``, ``consolidate_shard_weights`` rebuilds the full state dict from the files alone - for a convolutional
model whose units mix flattened and unflattened wrappers, widths that divide evenly and widths that need padding, a model
with a shared weight - and the result loads into a fresh wrapper that then computes the same loss.  Expert checkpoints that
were saved apart from the rest of the model consolidate with ``strict=False``."""
import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP

CPU = dict(compute_device=torch.device("cpu"))


def _conv_block(cin, cout):
    return nn.Sequential(nn.Conv2d(cin, cout, kernel_size=(3, 3)), nn.BatchNorm2d(cout), nn.ReLU())


class _ConvNet(nn.Module):
    def __init__(self, width, with_fsdp, group):
        super().__init__()
        torch.manual_seed(0)
        self.conv1 = _conv_block(3, width)
        self.conv2 = _conv_block(width, width // 2)
        self.conv3 = _conv_block(width // 2, width)
        self.pool = nn.AdaptiveAvgPool2d(output_size=(1, 1))
        self.flatten = nn.Flatten(start_dim=1)
        self.fc1 = nn.Linear(width, 2 * width)
        self.fc2 = nn.Linear(2 * width, 2 * width)
        self.fc3 = nn.Linear(2 * width, width + 1)
        self.fc4 = nn.Linear(width + 1, width)
        if with_fsdp:
            self.conv2 = FSDP(self.conv2, process_group=group, **CPU)
            self.conv3 = FSDP(self.conv3, process_group=group, flatten_parameters=False, **CPU)
            self.fc1 = FSDP(self.fc1, process_group=group, **CPU)
            self.fc3 = FSDP(self.fc3, process_group=group, flatten_parameters=False, **CPU)

    def forward(self, x):
        x = self.flatten(self.pool(self.conv3(self.conv2(self.conv1(x)))))
        x = torch.relu(self.fc1(x))
        x = torch.relu(self.fc2(x))
        x = torch.relu(self.fc3(x))
        return self.fc4(x)


def _make(width, with_fsdp, group, flatten=True):
    net = _ConvNet(width, with_fsdp, group)
    return FSDP(net, process_group=group, flatten_parameters=flatten, **CPU) if with_fsdp else net


def _conv_worker(rank, world, tmp, width, flatten):
    group = dist.new_group(list(range(world)))
    torch.manual_seed(1)
    x, target = torch.randn(4, 3, 12, 12), torch.zeros(4, width)
    model = _make(width, True, group, flatten)
    opt = torch.optim.SGD(model.parameters(), lr=1e-2)
    for _ in range(2):
        opt.zero_grad()
        nn.functional.mse_loss(model(x), target).backward()
        opt.step()
    torch.save({"weights": {k: v.cpu() for k, v in model.local_state_dict().items()}, "meta": model.local_metadata_dict()}, f"{tmp}/shard_{rank}.pt")
    dist.barrier()

    shards = [torch.load(f"{tmp}/shard_{r}.pt", weights_only=False) for r in range(world)]
    whole = FSDP.consolidate_shard_weights([s["weights"] for s in shards], [s["meta"] for s in shards])
    plain_sd = _make(width, False, group).state_dict()
    assert set(plain_sd.keys()) == set(whole.keys())
    assert all(whole[k].shape == v.shape for k, v in plain_sd.items())
    # the same tensors as the collective way of getting a full state dict
    for k, v in model.state_dict().items():
        torch.testing.assert_close(whole[k], v)
    without_buffers = FSDP.consolidate_shard_weights([s["weights"] for s in shards], [s["meta"] for s in shards], with_module_buffers=False)
    assert set(whole) - set(without_buffers) == {k for k in plain_sd if "running_" in k or "num_batches" in k}

    fresh = _make(width, True, group, flatten)
    fresh.load_state_dict(whole)
    model.eval()
    fresh.eval()
    with torch.no_grad():
        assert float(nn.functional.mse_loss(model(x), target)) == float(nn.functional.mse_loss(fresh(x), target))


@pytest.mark.parametrize("width", [16, 17])
@pytest.mark.parametrize("flatten", [True, False])
def test_convolutional_model_with_mixed_wrappers(tmp_path, width, flatten):
    spawn_ranks(_conv_worker, 2, (str(tmp_path), width, flatten), backend="gloo")


class _Tied(nn.Module):
    def __init__(self, wrap):
        super().__init__()
        torch.manual_seed(0)
        self.embed = nn.Embedding(19, 6)
        self.body = wrap(nn.Sequential(nn.Linear(6, 6), nn.Tanh()))
        self.out = nn.Linear(6, 19, bias=False)
        self.out.weight = self.embed.weight
        self.register_buffer("calls", torch.zeros(1))

    def forward(self, tokens):
        return self.out(self.body(self.embed(tokens)))


def _tied_worker(rank, world, tmp):
    model = FSDP(_Tied(lambda m: FSDP(m, **CPU)), **CPU)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    tokens = torch.randint(0, 19, (3, 4), generator=torch.Generator().manual_seed(rank))
    nn.functional.cross_entropy(model(tokens).flatten(0, 1), tokens.flatten()).backward()
    opt.step()
    torch.save({"weights": model.local_state_dict(), "meta": model.local_metadata_dict()}, f"{tmp}/s{rank}.pt")
    full = model.state_dict()
    dist.barrier()
    if rank == 0:
        shards = [torch.load(f"{tmp}/s{r}.pt", weights_only=False) for r in range(world)]
        whole = FSDP.consolidate_shard_weights([s["weights"] for s in shards], [s["meta"] for s in shards])
        assert set(whole) == set(full)
        for k, v in full.items():
            torch.testing.assert_close(whole[k], v)
        assert whole["out.weight"].data_ptr() == whole["embed.weight"].data_ptr()  # the tie survives
        with pytest.raises(ValueError):
            FSDP.consolidate_shard_weights([s["weights"] for s in shards], [shards[0]["meta"]])
        with pytest.raises(ValueError):
            FSDP.consolidate_shard_weights([], [])


def test_shared_weight_and_argument_checks(tmp_path):
    spawn_ranks(_tied_worker, 3, (str(tmp_path),), backend="gloo")


def test_expert_checkpoint_saved_apart_consolidates_without_strictness():
    path = "decoder.layers.1.moe_layer.experts.0"
    meta = {
        "param_metadata": [
            {"fsdp_path": "", "params": {"flat_param_0": {"names": ["missing"], "shapes": [(12, 4)], "numels": [48], "padding": 0}},
             "no_broadcast_optim_state": False, "shared_param_info": []},
            {"fsdp_path": path,
             "params": {"flat_param_0": {"names": ["fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"], "shapes": [(4, 4), (4,), (4, 4), (4,)],
                                         "numels": [16, 4, 16, 4], "padding": 0}},
             "no_broadcast_optim_state": True, "shared_param_info": []},
        ],
        "buffer_names": ["missing.buffer"],
    }
    weights = {f"{path}.flat_param_0": torch.randn(40, dtype=torch.float16)}
    whole = FSDP.consolidate_shard_weights([weights], [meta], strict=False)
    assert len(whole) == 4 and all(k.startswith(path) for k in whole)
    assert whole[f"{path}.fc1.weight"].shape == (4, 4) and whole[f"{path}.fc2.bias"].dtype == torch.float16
    with pytest.raises(KeyError):
        FSDP.consolidate_shard_weights([weights], [meta], strict=True)
