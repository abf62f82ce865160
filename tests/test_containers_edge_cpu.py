"""Edge cases of the container helpers (cases of the reference's tests/utils/test_containers.py): a single tensor instead of a
tuple, the packed format of non-tensor arguments (it is part of what checkpoint_wrapper saves for its replay), malformed
packs, mismatching keyword packs, in-place functions on packed RNN sequences, and state-dict key rewriting."""
from collections import OrderedDict

import pytest
import torch
from torch import nn

from fairscale_b200.internal.containers import apply_to_tensors, pack_kwargs, split_non_tensors, unpack_kwargs, unpack_non_tensors
from fairscale_b200.internal.state_dict import find_module_instances, replace_by_prefix_


def test_split_and_unpack_in_every_order():
    x, y = torch.Tensor([1]), torch.Tensor([2])
    tensors, packed = split_non_tensors(x)  # a single tensor instead of a tuple
    assert tensors == (x,) and packed is None
    tensors, packed = split_non_tensors((x, y, None, 3))
    assert tensors == (x, y) and packed == {"is_tensor": [True, True, False, False], "objects": [None, 3]}
    assert unpack_non_tensors(tensors, packed) == (x, y, None, 3)
    for mixed in ((None, 3, x, y), (None, 3), (x, y), (x, "a", y, "b")):
        tensors, packed = split_non_tensors(mixed)
        assert unpack_non_tensors(tensors, packed) == mixed
    assert unpack_non_tensors((x, y), None) == (x, y)
    with pytest.raises(AssertionError):
        unpack_non_tensors((x, y), set())  # the pack must be a dict
    with pytest.raises(AssertionError):
        unpack_non_tensors((x, y), {"is_tensor": [], "objects": []})  # ... that accounts for every tensor


def test_keyword_packs():
    keys, flat = pack_kwargs(1, 2, a=3, b=4)
    assert keys == ("a", "b") and flat == (1, 2, 3, 4)
    assert unpack_kwargs(keys, flat) == ((1, 2), {"a": 3, "b": 4})
    keys, flat = pack_kwargs(a=1)
    assert unpack_kwargs(keys, flat) == ((), {"a": 1})
    with pytest.raises(AssertionError):
        unpack_kwargs(["a", "b", "c", "d", "e"], (1, 2, 3, 4))  # more keys than values


def test_in_place_function_on_a_packed_sequence():
    rnn = nn.RNN(5, 5)
    x = nn.utils.rnn.pack_padded_sequence(torch.rand(5, 1, 5), torch.tensor([4], dtype=torch.int))
    out, _ = rnn(x)
    out = apply_to_tensors(lambda t: t.detach().fill_(0), out)
    padded, lengths = nn.utils.rnn.pad_packed_sequence(out)
    assert float(padded.sum()) == 0.0 and lengths.tolist() == [4]


def test_apply_visits_every_tensor_once_and_leaves_the_rest():
    seen = []
    data = OrderedDict(a=torch.ones(1), b=[torch.zeros(2), {"c": torch.ones(3), "d": 4}], e="text", f=None)
    out = apply_to_tensors(lambda t: seen.append(t.numel()) or t * 2, data)
    assert sorted(seen) == [1, 2, 3] and isinstance(out, OrderedDict)
    assert out["e"] == "text" and out["f"] is None and out["b"][1]["d"] == 4 and float(out["b"][1]["c"][0]) == 2.0


def test_state_dict_key_rewriting_and_instance_search():
    sd = OrderedDict([("abc.def", 1), ("abc.xyz", 2), ("abcdef", 3), ("x.abc.def", 4)])
    replace_by_prefix_(sd, "abc.", "new.")
    assert list(sd.keys()) == ["abcdef", "x.abc.def", "new.def", "new.xyz"] or set(sd) == {"abcdef", "x.abc.def", "new.def", "new.xyz"}
    replace_by_prefix_(sd, "new.", "")
    assert {"def", "xyz"} <= set(sd)
    with pytest.raises((ValueError, AssertionError)):
        replace_by_prefix_(sd, "same.", "same.")

    class Inner(nn.Module):
        pass

    net = nn.Sequential(nn.Linear(1, 1), nn.Sequential(Inner(), nn.Linear(1, 1)), Inner())
    found = find_module_instances(net, Inner)
    assert [name for name, _ in found] == ["1.0.", "2."] and all(isinstance(m, Inner) for _, m in found)
    assert find_module_instances(Inner(), Inner)[0][0] == ""
