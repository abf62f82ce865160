"""SlowMo: data parallelism with approximate averaging (LocalSGD or Stochastic Gradient Push) plus slow momentum.

Capability parity with fairscale/experimental/nn/data_parallel/gossip/distributed.py:57-1192: exact gradient
averaging inside a node, LocalSGD (parameter all-reduce every ``localsgd_frequency`` steps) or SGP (one push-sum /
push-pull gossip step per iteration) between nodes, the slow-momentum outer step every ``slowmo_frequency`` steps,
optionally sharded over ``slowmo_num_shards`` ranks, fp16 error feedback through ``fp32_params``.

Structure differences: gossip runs on the caller's thread as one batch of p2p operations (the reference's gossip
thread exists only for its disabled overlap mode); the sharded slow-momentum exchange works on ONE flat fp32
vector (a reduce to each shard owner, the momentum step as three fused foreach-free vector ops on the shard, a
broadcast back) rather than on per-parameter slices.
"""

from __future__ import annotations

from enum import Enum
import functools
import logging
import os
from typing import Any, Dict, Iterable, List, Optional, Tuple, Union, cast

import torch
import torch.distributed as dist
from torch.autograd import Variable
from torch.nn.modules import Module

from .gossiper import Gossiper, PushPull, PushSum
from .graph_manager import GraphManager
from .graph_manager import NPeerDynamicDirectedExponentialGraph as NPDDEGraph
from .mixing_manager import MixingManager, UniformMixing
from .utils import MultiProcessAdapter, communicate, create_process_group, flatten_tensors, group_by_dtype, unflatten_tensors
from .utils.cuda_metering import EventRecorder, create_event_recorder

HEARTBEAT_TIMEOUT = 300  # seconds a rank waits for a gossip partner (the process-group timeout enforces it)
BROADCAST_BUCKET_SIZE = 10 * 1024 * 1024


class SlowMoBaseAlgorithm(str, Enum):
    LOCALSGD = "localsgd"
    SGP = "sgp"


class SlowMoDistributedDataParallel(Module):
    """See the module docstring; argument names and defaults follow the reference constructor.

    Usage: ``loss.backward(); optimizer.step(); model.perform_slowmo(optimizer)``.
    """

    def __init__(self, module: torch.nn.Module, nprocs_per_node: int, broadcast_buffers: bool = True,
                 slowmo_base_algorithm: SlowMoBaseAlgorithm = SlowMoBaseAlgorithm.LOCALSGD, slowmo_momentum: float = 0.5,
                 slowmo_memory_efficient: bool = True, slowmo_frequency: int = 48, slowmo_lr: float = 1.0,
                 slowmo_num_shards: int = 32, localsgd_frequency: int = 3, graph: Optional[GraphManager] = None,
                 mixing: Optional[MixingManager] = None, push_sum: bool = True, overlap: bool = False, synch_freq: int = 0,
                 use_streams: bool = True, slowmo_sgp_average_params: bool = False, verbose: bool = False,
                 profile_mode: bool = False, process_rank: Optional[int] = None, process_world_size: Optional[int] = None,
                 global_group: Any = None, master_group: Any = None, local_node_group: Any = None,
                 comm_device: Optional[torch.device] = None) -> None:
        super().__init__()
        assert os.environ.get("NCCL_BLOCKING_WAIT", "0") == "0"
        assert nprocs_per_node >= 1
        assert not overlap, "overlap SGP is disabled"
        self.nprocs_per_node = nprocs_per_node
        if process_world_size is None or process_rank is None:
            assert dist.is_initialized()
            process_rank, process_world_size = dist.get_rank(), dist.get_world_size()
        self.process_rank, self.process_world_size = process_rank, process_world_size
        self.logger: Any = logging.getLogger(__name__)
        if verbose:
            self.logger.setLevel(logging.DEBUG)
            self.logger = MultiProcessAdapter(self.logger, {"process_num": process_rank})
        self._create_groups(global_group, master_group, local_node_group)
        self.module = module
        self.broadcast_buffers = broadcast_buffers
        self.module_buffers = list(module.buffers())
        self.broadcast_bucket_size = BROADCAST_BUCKET_SIZE
        first_dtype = next(module.parameters()).dtype
        if comm_device is None:
            comm_device = torch.device("cpu") if dist.get_backend() == "gloo" else torch.device("cuda", torch.cuda.current_device())
        self._cpu_comm = comm_device.type == "cpu"
        self.comm_device = comm_device
        self.profile_mode = profile_mode
        self.num_updates = 0
        self.slowmo = slowmo_lr != 1 or slowmo_momentum != 0
        self.slowmo_lr = slowmo_lr if self.slowmo else 1
        self.slowmo_momentum = slowmo_momentum if self.slowmo else 0
        self.slowmo_frequency = slowmo_frequency
        self.slowmo_sgp_average_params = slowmo_sgp_average_params
        self.localsgd = slowmo_base_algorithm == SlowMoBaseAlgorithm.LOCALSGD
        self.sgp = slowmo_base_algorithm == SlowMoBaseAlgorithm.SGP
        self.localsgd_frequency = localsgd_frequency
        self.overlap = False
        self.ef1: Optional[List[torch.Tensor]] = None
        self.global_momentum_buffers_initialized = False
        if self.master_group is None:
            assert self.localsgd or self.sgp
            self.localsgd = self.sgp = False
            self.logger.warning("Disabling LocalSGD and SGP since a local allreduce will suffice")
        if self.slowmo and not self.localsgd and not self.sgp:
            self.logger.warning("SlowMo is being used without LocalSGD and SGP")
        self.slowmo_memory_efficient = slowmo_memory_efficient
        self.slowmo_num_shards = min(process_world_size, slowmo_num_shards) if slowmo_memory_efficient else 1
        self.is_current_node_a_slowmo_shard = process_rank < self.slowmo_num_shards if slowmo_memory_efficient else True
        self.portion_start: Optional[int] = None
        if self.sgp:
            self._sgp_init(first_dtype, graph, mixing, push_sum)
        self.register_forward_pre_hook(self._forward_pre_hook)
        self._queued = False
        for p in module.parameters():
            if p.requires_grad:
                p.register_hook(self._grad_hook)

    # ------------------------------------------------------------------ groups
    def _create_groups(self, global_group: Any, master_group: Any, local_node_group: Any) -> None:
        n, rank, world = self.nprocs_per_node, self.process_rank, self.process_world_size
        assert world % n == 0, "total world size must be a multiple of nprocs_per_node"
        self.local_rank = rank % n
        self.logical_rank, self.logical_world_size = rank // n, world // n
        self.global_group = global_group if global_group is not None else create_process_group(list(range(world)))
        self.process_group = self.global_group
        if n == 1:
            self.local_node_group = None
        elif local_node_group is not None:
            self.local_node_group = local_node_group
        else:
            for node in range(self.logical_world_size):
                ranks = list(range(node * n, (node + 1) * n))
                g = create_process_group(ranks)
                if rank in ranks:
                    self.local_node_group = g
        if master_group is not None:
            self.master_group = master_group
        elif n > 1:
            masters = [i for i in range(world) if i % n == 0]
            self.master_group = create_process_group(masters) if len(masters) > 1 else None
        else:
            self.master_group = self.global_group if world > 1 else None

    def forward(self, *inputs: Any, **kwargs: Any) -> Any:
        return self.module(*inputs, **kwargs)

    # ------------------------------------------------------------------ hooks
    def _forward_pre_hook(self, *unused: Any) -> None:
        if self.broadcast_buffers and self.module_buffers:
            communicate(self.module_buffers, functools.partial(dist.broadcast, src=0, group=self.process_group))
        if self.sgp:
            self._sgp_unbias()

    def _grad_hook(self, grad: torch.Tensor) -> None:
        if not self._queued:
            self._queued = True
            Variable._execution_engine.queue_callback(self._after_backward)

    def _after_backward(self) -> None:
        self._queued = False
        if self.local_node_group is not None:
            grads = [p.grad for p in self.module.parameters() if p.requires_grad and p.grad is not None]
            torch._foreach_div_(grads, float(self.nprocs_per_node))
            communicate(grads, functools.partial(dist.all_reduce, group=self.local_node_group), None)
        if self.sgp:
            self._sgp_ps_numerator()

    # ------------------------------------------------------------------ schedule predicates
    def _should_perform_slowmo(self) -> bool:
        return self.slowmo and (self.num_updates + 1) % self.slowmo_frequency == 0

    def _should_perform_localsgd(self) -> bool:
        return self.localsgd and (self.num_updates + 1) % self.localsgd_frequency == 0

    def _skip_averaging_memory_efficient_slowmo(self) -> bool:
        return self.slowmo_memory_efficient and self._should_perform_slowmo()

    def _should_perform_sgp(self) -> bool:
        return self.sgp and not self._skip_averaging_memory_efficient_slowmo()

    def _should_allreduce_params(self) -> bool:
        return (self.sgp and self._should_perform_slowmo() and self.slowmo_sgp_average_params) or (
            self._should_perform_localsgd() and not self._skip_averaging_memory_efficient_slowmo()
        )

    def _should_use_error_feedback(self, pairs: List[Tuple[torch.Tensor, torch.Tensor]]) -> bool:
        return bool(pairs) and (self._should_perform_sgp() or self._should_allreduce_params())

    def _create_event_recorder(self, name: str) -> EventRecorder:
        return create_event_recorder(name, dummy=not self.profile_mode)

    # ------------------------------------------------------------------ fp16 master copies
    def _fp16_fp32_iterator(self, optimizer: Any, fp32_params: Any) -> Iterable[Tuple[torch.Tensor, torch.Tensor]]:
        stash = getattr(optimizer, "_amp_stash", None)
        if stash is not None and hasattr(stash, "fp16_groups"):
            for g16, g32 in zip(stash.fp16_groups, stash.fp32_from_fp16_groups):
                yield from zip(g16, g32)
        elif fp32_params is not None:
            if isinstance(fp32_params, dict):
                (fp32_params,) = list(fp32_params.values())
            if isinstance(fp32_params, list):
                for p, m in zip(self.parameters(), fp32_params):
                    yield p.view(-1), m
            else:
                off = 0
                for p in self.parameters():
                    yield p.view(-1), fp32_params[off : off + p.numel()]
                    off += p.numel()

    # ------------------------------------------------------------------ the outer step
    def perform_slowmo(self, optimizer: torch.optim.Optimizer, fp32_params: Optional[torch.Tensor] = None) -> None:
        """Call after ``optimizer.step()``: base-algorithm averaging for this iteration, then (when due) the slow
        momentum step.  ``fp32_params``: master copy (flat tensor, list, or 1-entry dict) when the model is fp16."""
        if not self.global_momentum_buffers_initialized:
            self._init_global_momentum_buffers(optimizer)
        pairs = list(self._fp16_fp32_iterator(optimizer, fp32_params))
        use_ef = self._should_use_error_feedback(pairs)
        with torch.no_grad():
            rec = self._create_event_recorder("Error feedback")
            if use_ef:  # keep in fp32 what the fp16 message cannot carry
                for p16, p32 in pairs:
                    if self._should_allreduce_params():
                        p16.div_(self.logical_world_size).mul_(self.logical_world_size)
                    p32 -= p16.float()
            rec.stop()
            rec = self._create_event_recorder("SGP")
            if self._should_perform_sgp() and not self._should_allreduce_params():
                self._sgp_gossip_step()
            rec.stop()
            rec = self._create_event_recorder("Localsgd communication time")
            if self._should_allreduce_params():
                params = list(self.parameters())
                torch._foreach_div_(params, float(self.logical_world_size))
                if self.process_rank % self.nprocs_per_node == 0:
                    communicate(params, functools.partial(dist.all_reduce, group=self.master_group), None)
            rec.stop()
            if self._should_perform_sgp() or self._should_allreduce_params():
                self._sync_params()
            if use_ef:
                for p16, p32 in pairs:
                    p32 += p16.float()
            rec = self._create_event_recorder("Slowmo")
            if self._should_perform_slowmo():
                self._global_momentum_step(optimizer)
            rec.stop()
            if pairs and (self._should_perform_sgp() or self._should_allreduce_params() or self._should_perform_slowmo()):
                for p16, p32 in pairs:
                    p16.copy_(p32)
        self.num_updates += 1

    def _sync_params(self) -> None:
        """Broadcast the node master's parameters inside the node."""
        if self.local_node_group is None:
            return
        communicate(list(self.module.parameters()),
                    functools.partial(dist.broadcast, src=self.logical_rank * self.nprocs_per_node, group=self.local_node_group))

    # ------------------------------------------------------------------ slow momentum
    def _optimizer_params(self, optimizer: Any) -> List[Tuple[torch.Tensor, float]]:
        return [(p, g["lr"]) for g in optimizer.param_groups for p in g["params"]]

    def _init_global_momentum_buffers(self, optimizer: Any) -> None:
        self.global_momentum_buffers_initialized = True
        if not self.slowmo:
            return
        plist = self._optimizer_params(optimizer)
        total = sum(p.numel() for p, _ in plist)
        assert all(p.dtype == torch.float32 for p, _ in plist), "slow momentum runs on fp32 (master) parameters"
        self._total_elements = total
        self.world_portion_length = (total + self.slowmo_num_shards - 1) // self.slowmo_num_shards
        if not self.is_current_node_a_slowmo_shard:
            return
        self.portion_start = self.process_rank * self.world_portion_length if self.slowmo_memory_efficient else 0
        self.portion_end = min((self.process_rank + 1) * self.world_portion_length, total) if self.slowmo_memory_efficient else total
        flat = flatten_tensors([p.detach() for p, _ in plist])
        self.old_params = flat[self.portion_start : self.portion_end].clone()
        self.global_momentum_buffer = torch.zeros_like(self.old_params)

    def _lr_vector(self, plist: List[Tuple[torch.Tensor, float]], start: int, end: int, like: torch.Tensor) -> Union[float, torch.Tensor]:
        lrs = {lr for _, lr in plist}
        if len(lrs) == 1:
            return lrs.pop()
        vec = torch.cat([torch.full((p.numel(),), lr, dtype=like.dtype, device=like.device) for p, lr in plist])
        return vec[start:end]

    def _global_momentum_step(self, optimizer: Any) -> None:
        if not self.slowmo:
            return
        plist = self._optimizer_params(optimizer)
        params = [p.detach() for p, _ in plist]
        flat = flatten_tensors(params)
        L = self.world_portion_length
        if self.slowmo_memory_efficient:
            flat.div_(self.process_world_size)
            works = [dist.reduce(flat[s * L : min((s + 1) * L, flat.numel())], dst=s, group=self.global_group, async_op=True)
                     for s in range(self.slowmo_num_shards) if s * L < flat.numel()]
            for w in works:
                w.wait()
        if self.is_current_node_a_slowmo_shard and self.portion_start is not None and self.portion_start < flat.numel():
            cur = flat[self.portion_start : self.portion_end]
            lr = self._lr_vector(plist, self.portion_start, self.portion_end, cur)
            # u <- beta * u + (x_old - x) / lr ;  x_old <- x_old - slowmo_lr * lr * u ;  x <- x_old
            self.global_momentum_buffer.mul_(self.slowmo_momentum).add_((self.old_params - cur) / lr)
            self.old_params.sub_(self.global_momentum_buffer * lr * self.slowmo_lr)
            cur.copy_(self.old_params)
        if self.slowmo_memory_efficient:
            works = [dist.broadcast(flat[s * L : min((s + 1) * L, flat.numel())], src=s, group=self.global_group, async_op=True)
                     for s in range(self.slowmo_num_shards) if s * L < flat.numel()]
            for w in works:
                w.wait()
        torch._foreach_copy_(params, unflatten_tensors(flat, params))

    # ------------------------------------------------------------------ SGP
    def _sgp_init(self, first_dtype: torch.dtype, graph: Optional[GraphManager], mixing: Optional[MixingManager], push_sum: bool) -> None:
        if graph is None:
            graph = NPDDEGraph(self.logical_rank, self.logical_world_size, self.nprocs_per_node, self.local_rank)
        if mixing is None:
            mixing = UniformMixing(graph, self.comm_device)
        self.graph, self.mixing, self.push_sum = graph, mixing, push_sum
        self.ps_weight = torch.ones(1, device=self.comm_device, dtype=first_dtype)
        self.is_sgp_ps_numerator = False
        self.gossip_enable = True
        self.lazy_mixing = mixing.is_regular()
        self.gossipers: Dict[torch.dtype, Gossiper] = {}
        if self.process_rank % self.nprocs_per_node == 0:
            cls = PushSum if push_sum else PushPull
            for dt, ps in group_by_dtype([p.detach() for p in self.module.parameters()]).items():
                self.gossipers[dt] = cls(flatten_tensors(ps).to(self.comm_device), graph=graph, device=self.comm_device, mixing=mixing,
                                         rank=self.process_rank, world_size=self.logical_world_size, group=self.global_group)

    def _sgp_gossip_step(self) -> None:
        """One push-sum iteration on the node masters (other ranks of the node receive the result by broadcast)."""
        if not self.gossip_enable or self.process_rank % self.nprocs_per_node != 0:
            return
        self._sgp_ps_numerator()
        ps_in = None
        lo = None
        for dt, ps in group_by_dtype([p.detach() for p in self.module.parameters()]).items():
            g = self.gossipers[dt]
            lo = g._mixing_manager.get_mixing_weights(False)["lo"].to(self.comm_device)
            if not self.lazy_mixing:
                torch._foreach_mul_(ps, float(lo))
            out = flatten_tensors(ps).to(self.comm_device)
            w = self.ps_weight * lo.to(self.ps_weight.dtype) if not self.lazy_mixing else self.ps_weight
            in_msg, ps_in = g.mix(out, w)
            recv = unflatten_tensors(in_msg.to(ps[0].device), ps)
            torch._foreach_add_(ps, recv)
            if self.lazy_mixing:
                torch._foreach_mul_(ps, float(lo))
        assert lo is not None and ps_in is not None
        if self.lazy_mixing:
            self.ps_weight = (self.ps_weight + ps_in.to(self.ps_weight.dtype)) * lo.to(self.ps_weight.dtype)
        else:
            self.ps_weight = self.ps_weight * lo.to(self.ps_weight.dtype) + ps_in.to(self.ps_weight.dtype)

    def _sgp_ps_numerator(self) -> None:
        """Parameters become the push-sum numerator (x * w)."""
        if not self.is_sgp_ps_numerator:
            if not self.lazy_mixing:
                with torch.no_grad():
                    for p in self.module.parameters():
                        p.mul_(self.ps_weight.to(p.device, p.dtype))
            self.is_sgp_ps_numerator = True

    def _sgp_unbias(self) -> None:
        """Parameters become the de-biased estimate (numerator / w) used by forward."""
        if self.is_sgp_ps_numerator:
            if not self.lazy_mixing:
                with torch.no_grad():
                    for p in self.module.parameters():
                        p.div_(self.ps_weight.to(p.device, p.dtype))
            self.is_sgp_ps_numerator = False

    # ------------------------------------------------------------------ module protocol
    def state_dict(self, *args: Any, **kwargs: Any) -> Dict[str, Any]:  # type: ignore[override]
        sd = super().state_dict(*args, **kwargs)
        if self.sgp:
            sd["ps_weight"] = self.ps_weight.cpu()
            sd["is_sgp_ps_numerator"] = self.is_sgp_ps_numerator
        return sd

    def load_state_dict(self, state_dict: Dict[str, Any], *args: Any, **kwargs: Any) -> Any:  # type: ignore[override]
        if self.sgp:
            state_dict = dict(state_dict)
            self.ps_weight = cast(torch.Tensor, state_dict.pop("ps_weight")).to(self.comm_device)
            self.is_sgp_ps_numerator = cast(bool, state_dict.pop("is_sgp_ps_numerator"))
        return super().load_state_dict(state_dict, *args, **kwargs)

    def train(self, mode: bool = True) -> "SlowMoDistributedDataParallel":
        super().train(mode)
        if self.sgp:
            self.gossip_enable = True
        return self

    def eval(self) -> "SlowMoDistributedDataParallel":
        super().eval()
        if self.sgp:
            self.gossip_enable = False
        return self
