"""Convert optimizer state between FSDP's sharded/flat form and the plain per-parameter form.

Format parity with fairscale/nn/data_parallel/fsdp_optim_utils.py:18-249: a consolidated
dict has ``state`` keyed by *original* parameter index, one ``param_groups`` entry, plus
``param_id_map`` (original index → FSDP-instance index, ``None`` if not collected) and
``uncollected_local_ids`` (instances whose state is rank-local, e.g. MoE experts).
"""

from __future__ import annotations

import copy
from typing import TYPE_CHECKING, Any, Dict, List, Optional, Tuple, cast

import torch

if TYPE_CHECKING:
    from .fully_sharded_data_parallel import FullyShardedDataParallel


def is_singleton_tensor(x: Any) -> bool:
    """0-dim tensor (e.g. Adam's ``step`` on recent torch)."""
    return torch.is_tensor(x) and x.dim() == 0


def flatten_optim_state_dict(sd: Dict) -> Dict:
    """Consolidated (per original parameter) → per FSDP instance, tensors concatenated flat.

    The result still holds *full* tensors; the caller slices this rank's shard.
    """
    id_map: Dict[int, Optional[int]] = sd["param_id_map"]
    instance_ids = {v for v in id_map.values() if v is not None}
    flat_pieces: Dict[int, Dict[str, List[torch.Tensor]]] = {i: {} for i in instance_ids} if sd["state"] else {}
    per_instance_other: Dict[int, Dict[str, Any]] = {i: {} for i in instance_ids}
    shared_scalars: Dict[str, Any] = {}

    for orig_id, buffers in sd["state"].items():
        inst = id_map[orig_id]
        for name, value in buffers.items():
            if is_singleton_tensor(value) or isinstance(value, list):
                per_instance_other[inst][name] = value
            elif torch.is_tensor(value):
                flat_pieces[inst].setdefault(name, []).append(value.reshape(-1))
            else:
                shared_scalars[name] = value

    new_state: Dict[int, Dict[str, Any]] = {}
    for inst, by_name in flat_pieces.items():
        merged: Dict[str, Any] = {name: torch.cat(parts) for name, parts in by_name.items()}
        merged.update(shared_scalars)
        merged.update(per_instance_other[inst])
        new_state[inst] = merged

    groups = copy.deepcopy(sd["param_groups"])
    # number of runs of equal instance id == number of instances that own parameters
    runs = 0
    prev: Any = object()
    for v in id_map.values():
        if v != prev:
            runs += 1
            prev = v
    for g in groups:
        g["params"] = list(range(runs))

    sd["state"] = new_state
    sd["param_groups"] = groups
    del sd["uncollected_local_ids"]
    del sd["param_id_map"]
    return sd


def check_param_counts_before_sharding(full_optim_state_dict: Dict, n_instances: int) -> None:
    n_saved = len(set(full_optim_state_dict["param_id_map"].values()))
    stateless = len(full_optim_state_dict["state"]) == 0
    assert stateless or n_instances == n_saved, (
        f"Including itself, this model has {n_instances} nested instances. When the optimizer state was saved "
        f"there were {n_saved}"
    )


def _scalar_state(gathered: Dict[int, Dict[str, List]], inst: int) -> Dict[str, Any]:
    """Non-tensor entries (``step`` …) must agree across ranks; keep one copy."""
    out: Dict[str, Any] = {}
    for name, per_rank in gathered[inst].items():
        if torch.is_tensor(per_rank[0]):
            continue
        if len(set(per_rank)) != 1:
            raise TypeError(f"Dont know how to consolidate optimizer param {name} with values {per_rank}")
        out[name] = per_rank[0]
    return out


def _unflatten_optim_state(
    gathered: Dict[int, Dict],
    instances: List["FullyShardedDataParallel"],
    world_pad_info: List[List[List[int]]],
    singleton_state: Dict[int, Dict],
) -> Tuple[Dict[int, Dict], Dict[int, Optional[int]]]:
    """Per-instance gathered shards → per original parameter state.

    ``world_pad_info[rank][instance][0]`` is the padding of that instance's flat shard on ``rank``.
    Returns ``(state, original index → instance index)``.
    """
    have_state = sorted(gathered.keys())
    pads = {i: [per_rank[i][0] for per_rank in world_pad_info] for i in gathered}
    scalars = {i: _scalar_state(gathered, i) for i in gathered}

    counts: List[int] = []
    for m in instances:
        counts.append(cast(int, m.num_params_managed) if m.flatten_parameters else len(m.non_shared_params()))

    orig_to_inst: Dict[int, Optional[int]] = {}
    inst_to_orig: Dict[int, List[int]] = {i: [] for i in have_state}
    nxt = 0
    for inst, n in enumerate(counts):
        for _ in range(n):
            orig_to_inst[nxt] = inst if inst in gathered else None
            if inst in gathered:
                inst_to_orig[inst].append(nxt)
            nxt += 1
    if not gathered:
        return {}, orig_to_inst

    first = have_state[0]
    out: Dict[int, Dict] = {
        g: copy.deepcopy(scalars[first]) for g, inst in orig_to_inst.items() if inst is not None
    }
    if scalars[first].keys() == gathered[first].keys():
        return out, orig_to_inst  # optimizer without tensor state (e.g. plain SGD)

    for inst in have_state:
        for name, per_rank in gathered[inst].items():
            if name in scalars[inst]:
                continue
            assert isinstance(per_rank, list), f"got {name}: {per_rank} for {inst}"
            unpadded = [t[:-pad] if pad > 0 else t for t, pad in zip(per_rank, pads[inst])]
            flat = torch.cat(unpadded)
            targets = sorted(inst_to_orig[inst])
            if instances[inst].flatten_parameters:
                for g, view in zip(targets, instances[inst].get_param_views([flat])):
                    assert name not in out[g], f"already added {name} to {g} {inst}"
                    out[g][name] = view
            else:
                assert len(targets) == 1, "Only support a single non-flatten parameter"
                out[targets[0]][name] = flat
        for g in inst_to_orig[inst]:
            out[g].update(singleton_state[inst])
    return out, orig_to_inst


def build_unflat_state_dict(
    instances: List["FullyShardedDataParallel"],
    world_pad_info: List[List[List[int]]],
    state: Dict[int, Dict[str, List[torch.Tensor]]],
    singleton_state: Dict[int, Dict[str, List[torch.Tensor]]],
    uncollected_opt_state: Dict[int, Dict],
    original_sd: Dict,
) -> Dict:
    """Rank-0 assembly of the consolidated optimizer state dict (as if FSDP were absent)."""
    assert all(len(s) == len(instances) for s in world_pad_info)
    assert all(len(s[0]) == 1 for s in world_pad_info)
    for inst, local in uncollected_opt_state.items():
        assert inst not in state
        state[inst] = {k: [v] for k, v in local.items() if not is_singleton_tensor(v)}
        singleton_state[inst] = {k: [v] for k, v in local.items() if is_singleton_tensor(v)}

    unflat, id_map = _unflatten_optim_state(state, instances, world_pad_info, singleton_state)
    groups = copy.deepcopy(original_sd["param_groups"])
    groups[0]["params"] = list(range(sum(cast(int, m.num_params_managed) for m in instances)))
    original_sd["state"] = dict(sorted(unflat.items()))
    original_sd["param_id_map"] = id_map
    original_sd["param_groups"] = groups
    original_sd["uncollected_local_ids"] = list(uncollected_opt_state.keys())
    return original_sd
