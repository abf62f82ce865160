"""ZeRO-1: optimizer state sharding (OSS).

API and checkpoint parity with fairscale/optim/oss.py:79-665: every rank owns a
greedy-by-size subset of the parameters, runs the wrapped optimizer on that subset only
and publishes the updated values to the other ranks; `consolidate_state_dict` /
`state_dict` / `load_state_dict` produce and accept dictionaries that are
interchangeable with those of the un-sharded optimizer.

Layout choice for B200: the parameters owned by one rank on one device live in one
flat, 16-byte aligned :class:`ParamBucket`, so the post-step publish is one collective
per owner (launch-latency bound on NVSwitch, not link bound) and a fused multi-tensor
optimizer can treat a whole shard as a single tensor.
"""

from __future__ import annotations

import copy
import io
import logging
from collections import OrderedDict
from itertools import chain
from math import inf
from typing import Any, Callable, Dict, List, Optional, Type, Union

import torch
import torch.distributed as dist
from torch.autograd import profiler
from torch.nn import Parameter
from torch.optim import SGD, Optimizer

from ..internal.params import calc_grad_norm, get_global_rank, recursive_copy_to_device
from ..nn.misc.param_bucket import ParamBucket
from ..parallel import comm, symm

__all__ = ["OSS"]

_params_t = Any


def _broadcast_object(
    obj: Any, src_rank: int, group: object = None, dist_device: torch.device = torch.device("cpu")
) -> Any:
    """Broadcast a picklable object as (length, bytes) tensors from global rank ``src_rank``.

    Fallback for ``dist.broadcast_object_list`` (selected with ``force_broadcast_object``).
    """
    group = dist.group.WORLD if group is None else group
    if dist.get_rank() == src_rank:
        stream = io.BytesIO()
        torch.save(obj, stream)
        payload = bytearray(stream.getbuffer())
        length = torch.tensor([len(payload)], dtype=torch.long, device=dist_device)
        body = torch.frombuffer(payload, dtype=torch.uint8).to(dist_device)
        dist.broadcast(length, src=src_rank, group=group)
        dist.broadcast(body, src=src_rank, group=group)
        return obj
    length = torch.zeros(1, dtype=torch.long, device=dist_device)
    dist.broadcast(length, src=src_rank, group=group)
    body = torch.empty(int(length.item()), dtype=torch.uint8, device=dist_device)
    dist.broadcast(body, src=src_rank, group=group)
    return torch.load(io.BytesIO(body.cpu().numpy().tobytes()), map_location=dist_device, weights_only=False)


class OSS(Optimizer):
    """Shard the state of ``optim`` over the ranks of ``group``.

    Args:
        params: parameters or param groups, as for any torch optimizer.
        optim: optimizer *class* to instantiate on the local shard (default SGD).
        group: process group (default WORLD).
        broadcast_buffer_size: deprecated, ignored.
        broadcast_fp16: publish updated parameters in fp16 to halve the traffic.
        force_broadcast_object: use tensor broadcasts instead of
            ``broadcast_object_list`` when exchanging optimizer state.
        **default: forwarded to ``optim``.
    """

    _instances = 0

    #: the wrapped optimizer, built on this rank's shard
    optim: Optimizer
    in_super_constructor: bool

    def __init__(
        self,
        params: _params_t,
        optim: Type[Optimizer] = SGD,
        group: Optional[Any] = None,
        broadcast_buffer_size: int = -1,
        broadcast_fp16: bool = False,
        force_broadcast_object: bool = False,
        **default: Any,
    ):
        self.in_super_constructor = True
        super().__init__(params, default)
        self.in_super_constructor = False
        self._instance = OSS._instances  # construction order is the same on every rank: names this optimizer's heap windows
        OSS._instances += 1

        # lazily (re)built partition caches; cleared by _clear_cache()
        self._cache_per_device: Dict[torch.device, List[List[Parameter]]] = OrderedDict()
        self._cache_param_rank: Dict[torch.Tensor, int] = {}
        self._partition_parameters: List[List[dict]] = []
        self._cache_param_index: Dict[int, int] = {}
        self._cache_local_params: Optional[List[torch.Tensor]] = None

        self._optim_defaults = default
        self._optim_constructor = optim

        self.group = group if group is not None else dist.group.WORLD
        self.world_size = dist.get_world_size(self.group)
        self.backend = dist.get_backend(self.group)
        self.rank = dist.get_rank(self.group)
        self.global_rank = get_global_rank(self.group, self.rank)
        self._local_to_global_rank = [get_global_rank(self.group, r) for r in range(self.world_size)]

        self.broadcast_fp16 = broadcast_fp16
        self.force_broadcast_object = force_broadcast_object
        self.buckets: Dict[torch.device, Dict[int, ParamBucket]] = {}
        self._unbucketed: Dict[torch.device, Dict[int, List[Parameter]]] = {}
        self._all_states: List[Dict[str, Any]] = []
        self._default_device = torch.device("cpu")

        self.refresh_trainable()

    # ------------------------------------------------------------------ partition
    def partition_parameters(self) -> List[List[dict]]:
        """Per-rank lists of param groups.

        Each parameter goes to the currently lightest rank; weight = numel (1 when
        frozen).  Element ``r`` holds shallow copies of the param groups restricted to
        rank ``r``'s parameters.  Every rank computes the full table because the
        publish step needs to know every owner.
        """
        if not self._partition_parameters:
            self._partition_parameters = [[] for _ in range(self.world_size)]
            load = [0] * self.world_size
            for group in self.param_groups:
                per_rank: List[List[Parameter]] = [[] for _ in range(self.world_size)]
                for p in group["params"]:
                    owner = load.index(min(load))
                    per_rank[owner].append(p)
                    load[owner] += p.numel() if p.requires_grad else 1
                for r, plist in enumerate(per_rank):
                    g = copy.copy(group)
                    g["params"] = plist
                    self._partition_parameters[r].append(g)
        return self._partition_parameters

    # ------------------------------------------------------------------ optimizer API
    def step(self, closure: Optional[Callable[[], float]] = None, **kwargs: Any) -> Optional[float]:
        """Step the local shard, then publish every shard to all ranks.  Extra kwargs go to the inner step."""
        OSS._sync_param_groups(self.param_groups, self.optim.param_groups)

        with profiler.record_function("fairscale::oss::refresh_trainable"):
            if self._default_device.type != self.param_groups[0]["params"][0].device.type:
                logging.info("OSS detected that the parameter changed devices, re-allocating buffers")
                self._clear_cache()
                self.refresh_trainable()

        with profiler.record_function("fairscale::oss::optim_step"):
            if closure is not None:
                loss = self.optim.step(closure=closure, **kwargs)  # type: ignore[call-arg]
            else:
                loss = self.optim.step(**kwargs)

        self._broadcast_params()
        OSS._sync_param_groups(self.optim.param_groups, self.param_groups)
        return loss

    def clip_grad_norm(
        self,
        max_norm: Union[float, int],
        norm_type: Union[float, int] = 2.0,
        filter_params_fn: Optional[Callable[[Any], Any]] = None,
    ) -> torch.Tensor:
        """Clip the *global* gradient norm; must be called on all ranks.

        Each rank only holds the gradients of its shard (with ShardedDataParallel), so
        the local norm is combined across ranks before the common scale is applied.  The combination runs over the WORLD
        group, not over this optimizer's group (as in the reference, fairscale/optim/oss.py:283-297): with model parallelism
        the ranks outside the data-parallel group hold other parameters of the same model.  Every rank of the world has to
        make the call.
        """
        max_norm = float(max_norm)
        norm_type = float(norm_type)
        with profiler.record_function("fairscale::oss::clip_grad_norm"):
            mine = self._local_params if filter_params_fn is None else filter_params_fn(self._local_params)
            local = calc_grad_norm(mine, norm_type).to(self._default_device)
            if norm_type == inf:
                total = local
                dist.all_reduce(total, op=dist.ReduceOp.MAX, group=dist.group.WORLD)
            else:
                total = local**norm_type
                dist.all_reduce(total)
                total = total ** (1.0 / norm_type)
            coef = torch.tensor(max_norm, dtype=total.dtype, device=total.device) / (total + 1e-6)
            if coef < 1:
                for device, per_rank in self._per_device_params.items():
                    scale = coef.to(device)
                    for p in per_rank[self.rank]:
                        if p.grad is not None:
                            p.grad.detach().mul_(scale)
        return total

    # ------------------------------------------------------------------ checkpointing
    def consolidate_state_dict(self, recipient_rank: int = 0) -> None:
        """Collect every rank's optimizer shard on ``recipient_rank`` (``-1``: on all ranks).

        Collective: call on all ranks.
        """
        OSS._sync_param_groups(self.param_groups, self.optim.param_groups)
        logging.debug("Pulling the sharded optimizer state from all replicas")
        self._all_states = []
        collect = recipient_rank in (self.rank, -1)
        must_send = self.rank != recipient_rank
        dist_device = torch.device("cuda") if self.backend == dist.Backend.NCCL else self._default_device
        cpu = torch.device("cpu")
        placeholder = lambda: torch.tensor([0], dtype=torch.uint8, device=dist_device)  # noqa: E731

        for r in range(self.world_size):
            src = self._local_to_global_rank[r]
            if r == self.rank:
                if collect:
                    self._all_states.append(
                        recursive_copy_to_device(self.optim.state_dict(), non_blocking=True, device=cpu)
                    )
                payload = self.optim.state_dict() if must_send else placeholder()
                self._exchange(payload, src, dist_device)
            else:
                received = self._exchange(placeholder(), src, dist_device)
                if collect:
                    self._all_states.append(recursive_copy_to_device(received, non_blocking=True, device=cpu))
                logging.debug("State from rank %s received", r)

    def _exchange(self, obj: Any, src_global_rank: int, dist_device: torch.device) -> Any:
        if self.force_broadcast_object:
            return _broadcast_object(obj, src_rank=src_global_rank, group=self.group, dist_device=dist_device)
        box = [obj]
        dist.broadcast_object_list(box, src=src_global_rank, group=self.group)
        return box[0]

    def state_dict(self, all_ranks: bool = False) -> Dict[str, Any]:
        """Global, torch-compatible optimizer state (sharding is not visible in it).

        Needs a prior :meth:`consolidate_state_dict` on the calling rank unless
        ``all_ranks=True`` (which then must be called on all ranks).
        """
        if not all_ranks and not self._all_states:
            raise RuntimeError(
                "Optimizer state has not been consolidated on this rank. "
                "Please call `consolidate_state_dict()` on all ranks beforehand if you meant to save the global state"
            )
        if all_ranks:
            self.consolidate_state_dict(recipient_rank=-1)

        merged = super().state_dict()
        for r, shard in enumerate(self._all_states):
            for local_group, owner_group in zip(shard["param_groups"], self.partition_parameters()[r]):
                for pos, local_idx in enumerate(local_group["params"]):
                    if local_idx in shard["state"]:
                        gid = self._param_to_index[id(owner_group["params"][pos])]
                        merged["state"][gid] = shard["state"][local_idx]
        merged["state"] = dict(sorted(merged["state"].items()))
        return merged

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        """Load a global state dict; only the entries of locally owned parameters are kept."""
        saved_ids = chain.from_iterable(g["params"] for g in state_dict["param_groups"])
        live_params = chain.from_iterable(g["params"] for g in self.param_groups)
        by_saved_id = dict(zip(saved_ids, live_params))

        for key, value in state_dict["state"].items():
            p = by_saved_id[key]
            if self._param_to_rank[p] != self.rank:
                state_dict["state"][key] = {}
            else:
                self.optim.state[p] = recursive_copy_to_device(value, non_blocking=True, device=p.device)

        super().load_state_dict(state_dict)
        OSS._sync_param_groups(state_dict["param_groups"], self.param_groups)
        OSS._sync_param_groups(self.param_groups, self.optim.param_groups)

    # ------------------------------------------------------------------ (re)configuration
    def refresh_trainable(self) -> None:
        """Rebuild the flat buffers after ``requires_grad`` changed on some parameters."""
        self._default_device = next(iter(self._per_device_params.keys()))
        if not hasattr(self, "optim"):
            self._clear_cache()
            self.optim = self._optim_constructor(self.partition_parameters()[self.rank], **self._optim_defaults)
            OSS._sync_param_groups(self.optim.param_groups, self.param_groups)
        self._setup_flat_buffers()

    def add_param_group(self, param_group: dict) -> None:
        """Add a param group on all ranks (collective in effect: call everywhere)."""
        super().add_param_group(param_group)
        if self.in_super_constructor:
            return
        self._clear_cache()
        mine = self.partition_parameters()[self.rank]
        if len(mine) == len(self.optim.param_groups) + 1:
            self.optim.add_param_group(mine[-1])
        self._setup_flat_buffers()

    # ------------------------------------------------------------------ cached views of the partition
    @property
    def _local_params(self) -> List[torch.Tensor]:
        """Locally owned parameters that currently have a gradient."""
        if self._cache_local_params is None:
            self._cache_local_params = [
                p for per_rank in self._per_device_params.values() for p in per_rank[self.rank] if p.grad is not None
            ]
        return self._cache_local_params

    @property
    def _param_to_index(self) -> Dict[int, int]:
        """``id(param)`` → index in the global (unsharded) optimizer numbering."""
        if not self._cache_param_index:
            flat = chain.from_iterable(g["params"] for g in self.param_groups)
            self._cache_param_index = {id(p): i for i, p in enumerate(flat)}
        return self._cache_param_index

    @property
    def _per_device_params(self) -> Dict[torch.device, List[List[Parameter]]]:
        """``device → [params owned by rank 0, rank 1, …]``, each list sorted by size."""
        if not self._cache_per_device:
            for group in self.param_groups:
                for p in group["params"]:
                    slot = self._cache_per_device.setdefault(p.device, [[] for _ in range(self.world_size)])
                    slot[self._param_to_rank[p]].append(p)
            for per_rank in self._cache_per_device.values():
                for plist in per_rank:
                    plist.sort(key=lambda t: t.numel())
        return self._cache_per_device

    @property
    def _param_to_rank(self) -> Dict[torch.Tensor, int]:
        if not self._cache_param_rank:
            for r, groups in enumerate(self.partition_parameters()):
                for g in groups:
                    for p in g["params"]:
                        self._cache_param_rank[p] = r
            logging.debug("OSS: parameters dispatched to ranks %s", list(self._cache_param_rank.values()))
        return self._cache_param_rank

    def _clear_cache(self) -> None:
        self._partition_parameters.clear()
        self._cache_per_device.clear()
        self._cache_param_rank.clear()
        self._cache_param_index.clear()
        self._cache_local_params = None

    @staticmethod
    def _sync_param_groups(source: List[Dict[Any, Any]], destination: List[Dict[Any, Any]]) -> None:
        """Copy scalar hyper-parameters (lr, momentum, …) between group lists so schedulers keep working."""
        for src, dst in zip(source, destination):
            for k, v in src.items():
                if k != "params":
                    dst[k] = v

    # ------------------------------------------------------------------ publish updated shards
    @torch.no_grad()
    def _broadcast_params(self) -> None:
        """Every owner broadcasts its flat bucket; stray (unbucketed) tensors follow one by one."""
        with profiler.record_function("fairscale::oss::refresh_trainable"):
            handles = []
            if self.broadcast_fp16:
                for device, per_owner in self.buckets.items():
                    for bucket in per_owner.values():
                        bucket.to(dtype=torch.float16, device=device, non_blocking=True, keep_param_alignment=False)

            for device, per_owner in self.buckets.items():
                for owner, bucket in per_owner.items():
                    handles.append(
                        comm.broadcast(
                            bucket.buffer, src=self._local_to_global_rank[owner], group=self.group, async_op=True
                        )
                    )
            for device, per_owner_list in self._unbucketed.items():
                for owner, plist in per_owner_list.items():
                    for p in plist:
                        handles.append(
                            comm.broadcast(
                                p.data, src=self._local_to_global_rank[owner], group=self.group, async_op=True
                            )
                        )
            for h in handles:
                if h is not None:
                    h.wait()

            if self.broadcast_fp16:
                for device, per_owner in self.buckets.items():
                    for bucket in per_owner.values():
                        bucket.to(dtype=torch.float32, device=device, non_blocking=True, keep_param_alignment=True)

    def _setup_flat_buffers(self) -> None:
        """Back the trainable parameters of each (device, owner) by one flat bucket.

        Frozen parameters are detached from any previous bucket.  Parameters whose dtype
        differs from the bucket's are published individually.
        """
        for device, per_rank in self._per_device_params.items():
            dev_buckets = self.buckets.setdefault(device, {})
            dev_loose = self._unbucketed.setdefault(device, {})
            for owner, plist in enumerate(per_rank):
                if not plist:
                    continue
                for p in plist:
                    if not p.requires_grad:
                        p.data = p.data.detach().clone()
                trainable = [p for p in plist if p.requires_grad]
                if not trainable:
                    dev_buckets.pop(owner, None)
                    dev_loose.pop(owner, None)
                    continue
                dtype = trainable[0].dtype
                members = [p for p in trainable if p.dtype == dtype]
                dev_loose[owner] = [p for p in trainable if p.dtype != dtype]
                align = max(1, 16 // members[0].element_size())
                # with an NVLink workspace the bucket lives in the symmetric heap: peers copy the owner's values out of it
                bucket = ParamBucket(
                    size=ParamBucket.required_size(members, align), dtype=dtype, device=device, align=align,
                    allocator=symm.heap_allocator(self.group, f"oss{self._instance}-param{owner}-{device}") if device.type == "cuda" else None,
                )
                for p in members:
                    bucket.add_param(p)
                dev_buckets[owner] = bucket

        live = set(self._per_device_params.keys())
        for stale in [d for d in self.buckets if d not in live]:
            self.buckets.pop(stale)
            self._unbucketed.pop(stale, None)
