"""Unit tests of the small building blocks: containers, sharding rule, state-dict key rewriting, version parsing, object
pickling, flat buckets and the flatten wrapper (single process, CPU)."""
from collections import OrderedDict, namedtuple

import pytest
import torch
from torch import nn

from fairscale_b200.internal.containers import apply_to_tensors, pack_kwargs, split_non_tensors, unpack_kwargs, unpack_non_tensors
from fairscale_b200.internal.object import pyobject_to_tensor, tensor_to_pyobject
from fairscale_b200.internal.parallel import chunk_and_pad
from fairscale_b200.internal.params import calc_grad_norm
from fairscale_b200.internal.state_dict import find_module_instances, replace_by_prefix_
from fairscale_b200.internal.version import torch_version
from fairscale_b200.nn.misc import FlattenParamsWrapper
from fairscale_b200.nn.misc.param_bucket import GradBucket, ParamBucket


def test_apply_to_tensors_keeps_container_types():
    Pair = namedtuple("Pair", ["a", "b"])
    data = {"x": torch.ones(2), "y": [torch.zeros(1), 3, "s"], "z": (torch.ones(1), Pair(torch.ones(3), None)), "w": {torch.ones(1)}}
    out = apply_to_tensors(lambda t: t + 1, data)
    assert isinstance(out["y"], list) and isinstance(out["z"], tuple) and isinstance(out["z"][1], Pair) and isinstance(out["w"], set)
    assert torch.equal(out["x"], torch.full((2,), 2.0)) and out["y"][1:] == [3, "s"] and out["z"][1].b is None
    packed = nn.utils.rnn.pack_sequence([torch.ones(3), torch.ones(2)])
    assert torch.equal(apply_to_tensors(lambda t: t * 2, packed).data, packed.data * 2)


def test_pack_unpack_kwargs_and_non_tensors():
    keys, flat = pack_kwargs(1, 2, a=3, b=4)
    assert keys == ("a", "b") and flat == (1, 2, 3, 4)
    assert unpack_kwargs(keys, flat) == ((1, 2), {"a": 3, "b": 4})
    assert unpack_kwargs((), (1, 2)) == ((1, 2), {})
    x, y = torch.ones(1), torch.zeros(2)
    tensors, packed = split_non_tensors((x, None, y, "str"))
    assert len(tensors) == 2 and tensors[0] is x and tensors[1] is y
    back = unpack_non_tensors(tensors, packed)
    assert back[0] is x and back[1] is None and back[2] is y and back[3] == "str"
    only, packed = split_non_tensors((x, y))
    assert unpack_non_tensors(only, packed) == (x, y)


@pytest.mark.parametrize("numel,chunks", [(10, 4), (3, 8), (16, 4), (1, 2)])
def test_chunk_and_pad_is_the_sharding_rule(numel, chunks):
    t = torch.arange(1, numel + 1, dtype=torch.float32)
    parts = chunk_and_pad(t, chunks)
    assert len(parts) == chunks and len({p.numel() for p in parts}) == 1
    ref = list(t.chunk(chunks))
    size = ref[0].numel()
    assert parts[0].numel() == size
    glued = torch.cat(parts)
    assert torch.equal(glued[:numel], t) and torch.count_nonzero(glued[numel:]) == 0


def test_replace_by_prefix_and_find_instances():
    sd = OrderedDict([("layer.a", 1), ("layer.b", 2), ("other.layer.c", 3)])
    replace_by_prefix_(sd, "layer.", "module.layer.")
    assert set(sd) == {"module.layer.a", "module.layer.b", "other.layer.c"}
    with pytest.raises(ValueError):
        replace_by_prefix_(sd, "x", "x")
    model = nn.Sequential(nn.Linear(2, 2), nn.Sequential(nn.ReLU(), nn.Linear(2, 2)))
    found = find_module_instances(model, nn.Linear)
    assert [n for n, _ in found] == ["0.", "1.1."]


def test_version_and_object_round_trip():
    assert torch_version("1.13.1") == (1, 13, 1)
    assert torch_version("2.11.0+cu128")[:2] == (2, 11)
    assert torch_version("2.0.0a0+git1234")[:3] == (2, 0, 0)
    obj = {"a": [1, 2, 3], "b": "text"}
    t = pyobject_to_tensor(obj, fixed_buffer_size=512)
    assert t.dtype == torch.uint8 and t.numel() == 512
    assert tensor_to_pyobject(t) == obj
    with pytest.raises(Exception):
        pyobject_to_tensor(list(range(1000)), fixed_buffer_size=16)


def test_calc_grad_norm():
    ps = [nn.Parameter(torch.ones(3)), nn.Parameter(torch.ones(2)), nn.Parameter(torch.ones(1))]
    ps[0].grad, ps[1].grad = torch.full((3,), 2.0), torch.full((2,), -3.0)
    assert torch.isclose(calc_grad_norm(ps, 2.0), torch.tensor(30.0).sqrt())
    assert calc_grad_norm(ps, float("inf")) == 3.0
    assert calc_grad_norm([ps[2]], 2.0) == 0.0
    # a bare tensor, another order, an integer order, and the dtype of the first parameter that counts
    assert torch.isclose(calc_grad_norm(ps[0], 1), torch.tensor(6.0))
    assert torch.isclose(calc_grad_norm(ps, 1.0), torch.tensor(12.0))
    half = nn.Parameter(torch.ones(4, dtype=torch.bfloat16))
    half.grad = torch.full((4,), 0.5, dtype=torch.bfloat16)
    norm = calc_grad_norm([ps[2], half, ps[0]], 2.0)  # ps[2] has no gradient
    assert norm.dtype == torch.bfloat16 and torch.isclose(norm.float(), torch.tensor(13.0).sqrt(), rtol=1e-2)
    assert calc_grad_norm(iter(ps), 2.0) > 5  # any iterable of parameters


def test_recursive_copy_to_device_walks_containers_and_leaves_the_rest():
    from collections import OrderedDict, namedtuple

    from fairscale_b200.internal.params import get_global_rank, recursive_copy_to_device

    Pair = namedtuple("Pair", "a b")
    value = {"t": torch.ones(2, dtype=torch.float64), "l": [torch.zeros(1), "text", 3], "tup": (torch.ones(1), None),
             "od": OrderedDict(x=torch.ones(1)), "np": Pair(torch.ones(1), 2)}
    moved = recursive_copy_to_device(value, non_blocking=False, device=torch.device("cpu"))
    assert moved["t"].dtype == torch.float64 and moved["l"][1:] == ["text", 3] and moved["tup"][1] is None
    assert isinstance(moved["l"], list) and isinstance(moved["tup"], tuple) and isinstance(moved["od"], dict)
    assert isinstance(moved["np"], tuple) and torch.equal(moved["np"][0], torch.ones(1)) and moved["np"][1] == 2
    assert recursive_copy_to_device(5, non_blocking=True, device=torch.device("cpu")) == 5
    assert get_global_rank(None, 3) == 3  # no group: ranks are already global


def test_param_and_grad_buckets():
    params = [nn.Parameter(torch.randn(3, 2)), nn.Parameter(torch.randn(5))]
    before = [p.detach().clone() for p in params]
    bucket = ParamBucket(size=11, dtype=torch.float32, device=torch.device("cpu"))
    for p in params:
        bucket.add_param(p)
    with pytest.raises(AssertionError):
        bucket.add_param(params[0])
    assert all(torch.equal(p, b) for p, b in zip(params, before))
    bucket.buffer.zero_()  # parameters are views of the flat buffer
    assert all(torch.count_nonzero(p) == 0 for p in params)

    gb = GradBucket(size=12, dtype=torch.float32, device=torch.device("cpu"), destination=1)  # an exact fit is refused, as in the reference
    for p in params:
        assert gb.can_add_grad_view(p)
        gb.add_grad(p)
    assert gb.destination == 1 and not gb.all_checked_in
    params[0].grad.fill_(1.0)
    params[1].grad.fill_(2.0)
    assert gb.buffer[:6].eq(1).all() and gb.buffer[6:11].eq(2).all()
    gb.collapse()  # the flat storage is released, the gradients are dropped
    assert all(p.grad is None for p in params)
    gb.rebuild()
    assert all(p.grad is not None and p.grad.shape == p.shape for p in params)
    gb.shrink()
    assert gb.buffer.numel() == 11


def test_flatten_params_wrapper_views_and_state_dict():
    torch.manual_seed(0)
    shared = nn.Linear(4, 4)
    model = nn.Sequential(shared, nn.ReLU(), nn.Linear(4, 4), shared)
    ref = [p.detach().clone() for p in model.parameters()]
    x = torch.randn(2, 4)
    expect = model(x)
    n_unique = sum(p.numel() for p in model.parameters())
    wrapped = FlattenParamsWrapper(model)
    flat = [p for p in wrapped.parameters()]
    assert len(flat) == 1 and flat[0].numel() == n_unique and flat[0].dim() == 1
    assert torch.allclose(wrapped(x), expect)
    wrapped(x).sum().backward()
    assert flat[0].grad is not None and flat[0].grad.shape == flat[0].shape
    # the unflattened state dict keeps the original names; the flat one has the single flat parameter
    names = set(wrapped.state_dict().keys())
    assert {"0.weight", "0.bias", "2.weight", "2.bias"} <= names
    assert list(wrapped.flat_state_dict().keys()) == ["flat_param_0"]
    with wrapped.unflatten_params():
        got = [p.detach().clone() for p in wrapped.module.parameters()]
    assert all(torch.equal(a, b) for a, b in zip(got, ref))
    # loading an unflattened state dict into a fresh wrapper reproduces the outputs
    other = FlattenParamsWrapper(nn.Sequential(nn.Linear(4, 4), nn.ReLU(), nn.Linear(4, 4), nn.Identity()))
    sd = {k: v for k, v in wrapped.state_dict().items() if not k.startswith("3.")}
    other.load_state_dict(sd, strict=False)
    with other.unflatten_params():
        assert torch.equal(other.module[0].weight, ref[0])


def test_flatten_params_wrapper_param_groups():
    model = nn.Sequential(nn.Linear(3, 3), nn.Linear(3, 3), nn.Linear(3, 2))
    group0 = list(model[0].parameters())
    group1 = list(model[2].parameters())
    wrapped = FlattenParamsWrapper(model, param_list=[group0, group1])
    names = [n for n, _ in wrapped.named_parameters()]
    assert sum(n.startswith("flat_param_") for n in names) == 2
    assert len(names) == 4  # two flat parameters + the untouched middle layer's weight and bias
    views = wrapped.flat_params[0].get_param_views()
    assert [v.shape for v in views] == [torch.Size([3, 3]), torch.Size([3])]
    meta = wrapped.flat_params[1].metadata()
    assert list(meta[1]) == [torch.Size([2, 3]), torch.Size([2])] and list(meta[2]) == [6, 2]
