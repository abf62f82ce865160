"""ZeRO-2: gradient sharding on top of :class:`fairscale_b200.optim.OSS`.

API parity with fairscale/nn/data_parallel/sharded_ddp.py:33-670.  During backward,
each gradient (or a flat bucket of gradients with the same owner) is sum-reduced to the
rank whose optimizer shard owns the parameter; every other rank drops it.

Implementation notes:

* hooks are ``Tensor.register_post_accumulate_grad_hook`` callbacks (one small object
  per parameter) rather than closures on grad-accumulator nodes;
* the end-of-backward flush is queued on the autograd engine, so ``loss.backward()``
  returns with every reduction finished;
* scaling by ``1/world`` happens *before* the sum, as in the reference
  (sharded_ddp.py:424,471), which keeps fp32 results identical to DDP for power-of-two
  world sizes.
"""

from __future__ import annotations

import contextlib
import logging
from collections import deque
from itertools import chain
from typing import TYPE_CHECKING, Any, Callable, Deque, Dict, Generator, List, Optional, Union

import torch
import torch.distributed as dist
from torch import nn
from torch.autograd import Variable, profiler

from ...internal.params import Workhandle, get_global_rank
from ...parallel import comm, symm
from ..misc.param_bucket import GradBucket


if TYPE_CHECKING:
    from ...optim.oss import OSS


def _trainable(p: torch.Tensor) -> bool:
    return p.requires_grad


class _ReduceHook:
    """Post-accumulate hook of one parameter: reduce it now, or check it into its bucket."""

    __slots__ = ("owner", "index", "param", "dst_rank", "bucketed")

    def __init__(self, owner: "ShardedDataParallel", index: int, param: torch.Tensor, dst_rank: int, bucketed: bool):
        self.owner = owner
        self.index = index
        self.param = param
        self.dst_rank = dst_rank
        self.bucketed = bucketed

    @torch.no_grad()
    def __call__(self, *_: Any) -> None:
        sdp, idx, param = self.owner, self.index, self.param
        if sdp._should_accumulate_grads or not sdp._grad_to_be_reduced[idx]:
            return
        assert param.grad is not None, "Reducing gradients during backward pass, cannot be None"
        sdp._ensure_flush_queued()
        sdp._grad_to_be_reduced[idx] = False

        if self.bucketed:
            bucket = sdp._buckets[param.device][self.dst_rank]
            bucket.readopt_grad(param)  # a gradient dropped by zero_grad(set_to_none=True) comes back as a private tensor
            bucket.params_checked_in += 1
            if bucket.all_checked_in:
                sdp._send_bucket(bucket)
        else:
            param.grad.mul_(sdp._world_size_scaling)
            if sdp._reduce_fp16:
                param.grad.data = param.grad.data.half()
            dst_global = sdp._local_to_global_rank[self.dst_rank]
            keep = dst_global == sdp._global_rank

            def cleanup(p: torch.Tensor = param, keep: bool = keep) -> None:
                if not keep:
                    p.grad = None
                else:
                    assert p.grad is not None
                    p.grad.data = p.grad.data.to(dtype=p.dtype)

            handle = comm.reduce(param.grad.data, dst=dst_global, group=sdp._process_group, async_op=True)
            sdp._work_handles.append(Workhandle(handle=handle, callback=cleanup))
        sdp._try_consume_work_handle()


class ShardedDataParallel(nn.Module):
    _instances = 0  # construction order is the same on every rank: names the heap windows of this wrapper's buckets
    """Wrap ``module`` so its gradients are reduced to the owning rank of ``sharded_optimizer``.

    Args:
        module: model to train.
        sharded_optimizer: one :class:`OSS` or a list of them covering the parameters.
        process_group: group for the reductions (default WORLD).
        broadcast_buffers: broadcast module buffers from rank 0 before each forward.
        sync_models_at_startup: broadcast the full model state from rank 0 at construction.
        reduce_buffer_size: element capacity of each per-owner gradient bucket;
            0 disables bucketing.
        auto_refresh_trainable: re-detect ``requires_grad`` changes every forward.
        reduce_fp16: reduce in fp16 (ignored when bucketing is on).
        warn_on_trainable_params_changed: log when trainability changed.
    """

    def __init__(
        self,
        module: nn.Module,
        sharded_optimizer: Union["OSS", List["OSS"]],
        process_group: Any = None,
        broadcast_buffers: bool = True,
        sync_models_at_startup: bool = True,
        reduce_buffer_size: int = 2**23,
        auto_refresh_trainable: bool = True,
        reduce_fp16: bool = False,
        warn_on_trainable_params_changed: bool = True,
    ):
        super().__init__()
        self._instance = ShardedDataParallel._instances
        ShardedDataParallel._instances += 1
        self.module = module
        self._sharded_optimizers = sharded_optimizer if isinstance(sharded_optimizer, list) else [sharded_optimizer]
        self._enable_broadcast_buffers = broadcast_buffers
        self._auto_refresh_trainable = auto_refresh_trainable
        self._reduce_fp16 = reduce_fp16
        if reduce_buffer_size > 0 and reduce_fp16:
            self._reduce_fp16 = False
            logging.warning(
                "fp16 gradient reduction is not compatible with reduction buffers, which are requested. "
                "fp16 grad reduction is deactivated."
            )
        self._warn_on_trainable_params_changed = warn_on_trainable_params_changed

        self._should_accumulate_grads = False
        self._accumulate_grads_flipped = False

        self._process_group = process_group if process_group is not None else dist.group.WORLD
        world = dist.get_world_size(self._process_group)
        self._backend = dist.get_backend(self._process_group)
        self._world_size_scaling = 1.0 / world
        self._reference_global_rank = get_global_rank(self._process_group, 0)
        self._rank = dist.get_rank(self._process_group)
        self._global_rank = get_global_rank(self._process_group, self._rank)
        self._local_to_global_rank = [get_global_rank(self._process_group, r) for r in range(world)]

        # DDP-compatible attributes
        device_types = {p.device.type for p in self.module.parameters()}
        self.is_multi_device_module = len({p.device for p in self.module.parameters()}) > 1
        assert len(device_types) == 1, (
            "ShardedDataParallel's input module must be on the same type of devices, "
            f"but input module parameters are located on {device_types} different device types."
        )
        self.device_type = next(iter(device_types))

        self._all_params: List[torch.Tensor] = [
            p
            for optim in self._sharded_optimizers
            for per_rank in optim._per_device_params.values()
            for plist in per_rank
            for p in plist
        ]
        self._trainable_params: List[torch.Tensor] = []
        self._grad_to_be_reduced: List[bool] = []
        self._trainable_param_to_rank: Dict[torch.Tensor, int] = {}
        self._reference_trainable_mask = [_trainable(p) for p in self._all_params]

        model_size = sum(p.numel() for p in self.module.parameters())
        self._buffer_max_size = min(reduce_buffer_size, model_size)
        if world == 1:
            self._buffer_max_size = 0
            logging.info("Training is not really distributed, single rank. Deactivating buckets")
        logging.info(
            "ShardedDDP bucket size: {:.2f}M parameters, model size {:.2f}M parameters".format(
                self._buffer_max_size / 2**20, model_size / 2**20
            )
        )
        self._use_buckets = self._buffer_max_size > 0
        self._buckets: Dict[torch.device, Dict[int, GradBucket]] = {}
        self._should_bucket_grad: List[bool] = []
        self._bucket_list: List[GradBucket] = []

        self._grad_hooks: List[Any] = []
        self._manual_reduce: List[Callable] = []

        self._passing_sync_batchnorm_handle(self.module)
        if sync_models_at_startup:
            self._sync_params_and_buffers()

        self._work_handles: Deque[Workhandle] = deque()
        self._bucket_flush_callback_set = False

    # ------------------------------------------------------------------ forward
    def forward(self, *inputs: Any, **kwargs: Any) -> Any:
        with profiler.record_function("fairscale::sdp::forward"):
            needs_setup = len(self._grad_hooks) == 0 and self.training
            if self._auto_refresh_trainable:
                needs_setup |= self._detect_train_change()
            if needs_setup:
                self.refresh_trainable()
            if self._enable_broadcast_buffers and not self._should_accumulate_grads:
                self.sync_buffers(blocking=True)
            self._clear_counters()
            return self.module(*inputs, **kwargs)

    def to(  # type: ignore[override]
        self, device: Optional[Union[str, torch.device]], dtype: Optional[torch.dtype] = None, non_blocking: bool = False
    ) -> "ShardedDataParallel":
        """Cast / move within the same device type.  Changing device type is refused because the
        optimizer shards would be left pointing at the old storage."""
        if isinstance(device, str):
            device = torch.device(device)
        assert (
            device is None or len(self._buckets) == 0 or device.type in {d.type for d in self._buckets}
        ), "Changing devices is not supported, because this would break OSSs state"
        assert len(self._buckets) < 2, (
            "Several devices specified to begin with, incompatible with setting a single device here"
        )
        self.module.to(device=device, dtype=dtype, non_blocking=non_blocking)
        self.refresh_trainable()
        return self

    def refresh_trainable(self) -> None:
        """Recompute owners, buckets and hooks after trainability changed."""
        if any(self._grad_to_be_reduced):
            logging.warning(
                "Grads waiting to be reduced. If this is on purpose (grad accumulation), please use a no_sync() context"
            )
        with profiler.record_function("fairscale::sdp::refresh_trainable"):
            # A parameter that has just been frozen may still carry last step's gradient as a view of a bucket that is
            # about to be rebuilt without it; zero_grad() only visits trainable parameters, so that stale value would be
            # applied by the optimizer again and again.  (A gradient set by hand on a frozen parameter is left alone.)
            for bucket in self._bucket_list:
                for p in bucket._params:
                    if not p.requires_grad and p.grad is not None:
                        p.grad = None
            self._trainable_params = sorted((p for p in self._all_params if p.requires_grad), key=lambda t: t.numel())
            self._trainable_param_to_rank = {}
            for optim in self._sharded_optimizers:
                optim.refresh_trainable()
                for per_rank in optim._per_device_params.values():
                    for plist in per_rank:
                        for p in plist:
                            if p.requires_grad:
                                self._trainable_param_to_rank[p] = optim._param_to_rank[p]
            self._setup_bucket_strategy()
            self._setup_backward_hooks()

    def reduce(self) -> None:
        """Reduce the accumulated gradients by hand (after backward passes under :meth:`no_sync`)."""
        assert any(self._grad_to_be_reduced), (
            "No grads waiting to be reduced, maybe that this was called twice or there was no BW pass ?"
        )
        self._bucket_flush_callback_set = True  # the flush is run below, not by the engine
        for fn in self._manual_reduce:
            fn()
        self._flush_reduce_calls()

    @torch.no_grad()
    def sync_buffers(self, blocking: bool = False) -> None:
        """Broadcast module buffers (e.g. BatchNorm statistics) from the group's rank 0."""
        with profiler.record_function("fairscale::sdp::sync_buffers"):
            handles = [
                comm.broadcast(b.data, self._reference_global_rank, self._process_group, async_op=True)
                for b in self.module.buffers(recurse=True)
            ]
            handles = [h for h in handles if h is not None]
            if blocking and handles:
                if self._backend != dist.Backend.NCCL:
                    for h in handles:
                        h.wait()
                else:
                    handles[-1].wait()  # NCCL ops complete in issue order on one stream

    def zero_grad(self, set_to_none: bool = False) -> None:
        """Zero (or drop) gradients; bucketed gradients stay views of their bucket and are zeroed."""
        for i, p in enumerate(self._trainable_params):
            bucketed = bool(self._should_bucket_grad) and self._should_bucket_grad[i]
            if set_to_none and not bucketed:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()
        for bucket in self._bucket_list:
            bucket.zero()

    def __getattr__(self, name: str) -> Any:
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)

    @contextlib.contextmanager
    def no_sync(self) -> Generator:
        """Accumulate gradients locally; nothing is reduced inside the context."""
        previous = self._should_accumulate_grads
        self._should_accumulate_grads = True
        yield
        self._accumulate_grads_flipped = self._should_accumulate_grads != previous
        self._should_accumulate_grads = previous

    # ------------------------------------------------------------------ internals
    @torch.no_grad()
    def _clear_counters(self) -> None:
        if self.training:
            self._grad_to_be_reduced = [True] * len(self._trainable_params)
        self._bucket_flush_callback_set = False
        if self._use_buckets:
            for bucket in self._bucket_list:
                bucket.reset_checked_in()
        if not self._should_accumulate_grads:
            self._accumulate_grads_flipped = False

    def _ensure_flush_queued(self) -> None:
        if not self._bucket_flush_callback_set:
            Variable._execution_engine.queue_callback(self._flush_reduce_calls)
            self._bucket_flush_callback_set = True

    def _send_bucket(self, bucket: GradBucket) -> None:
        assert bucket.buffer is not None
        bucket.buffer.mul_(self._world_size_scaling)
        bucket.sent = True
        handle = comm.reduce(bucket.buffer, dst=bucket.destination, group=self._process_group, async_op=True)
        self._work_handles.append(Workhandle(handle=handle, callback=None))

    def _get_reduce_fn(self, index: int, param: torch.Tensor, dst_rank: int) -> Callable:
        bucketed = self._use_buckets and self._should_bucket_grad[index]
        return _ReduceHook(self, index, param, dst_rank, bucketed)

    def _setup_backward_hooks(self) -> None:
        with profiler.record_function("fairscale::sdp::setup_backward_hooks"):
            while self._grad_hooks:
                self._grad_hooks.pop().remove()
            self._manual_reduce = []
            if not self.training:
                return
            for index, p in enumerate(self._trainable_params):
                if p.grad is not None and p.grad.requires_grad:
                    raise RuntimeError("ShardedDataParallel only works with gradients that don't require grad")
                fn = self._get_reduce_fn(index, p, self._trainable_param_to_rank[p])
                self._grad_hooks.append(p.register_post_accumulate_grad_hook(fn))
                self._manual_reduce.append(fn)

    @torch.no_grad()
    def _sync_params_and_buffers(self) -> None:
        handles = [
            comm.broadcast(t, src=self._reference_global_rank, group=self._process_group, async_op=True)
            for t in self.module.state_dict().values()
        ]
        handles = [h for h in handles if h is not None]
        if self._backend != dist.Backend.NCCL:
            for h in handles:
                h.wait()
        elif handles:
            handles[-1].wait()

    def _passing_sync_batchnorm_handle(self, module: nn.Module) -> None:
        for layer in module.modules():
            if isinstance(layer, torch.nn.modules.SyncBatchNorm) and hasattr(layer, "_specify_ddp_gpu_num"):
                assert self.device_type != "cpu", "SyncBatchNorm layers only work with GPU modules"
                layer._specify_ddp_gpu_num(1)  # type: ignore[attr-defined]

    def _setup_bucket_strategy(self) -> None:
        """One unsharded gradient bucket per (device, owner); small tensors first (params are sorted by size)."""
        with profiler.record_function("fairscale::sdp::setup_buckets"):
            if not self._use_buckets:
                return
            self._buckets = {}
            self._should_bucket_grad = [False] * len(self._trainable_params)
            for i, p in enumerate(self._trainable_params):
                dst = self._trainable_param_to_rank[p]
                per_dev = self._buckets.setdefault(p.device, {})
                if dst not in per_dev:
                    # with an NVLink workspace the bucket lives in the symmetric heap: its owner pulls the peers' copies
                    per_dev[dst] = GradBucket(
                        self._buffer_max_size,
                        dtype=p.dtype,
                        device=p.device,
                        destination=self._local_to_global_rank[dst],
                        align=max(1, 16 // p.element_size()),
                        allocator=symm.heap_allocator(self._process_group, f"sdp{self._instance}-grad{dst}") if p.is_cuda else None,
                    )
                bucket = per_dev[dst]
                if bucket.buffer.dtype == p.dtype and bucket.can_add_grad_view(p):
                    bucket.add_grad(p)
                    self._should_bucket_grad[i] = True
            self._bucket_list = list(chain.from_iterable(d.values() for d in self._buckets.values()))
            for bucket in self._bucket_list:
                if bucket._params:
                    bucket.shrink()

    def _consume_work_handles(self) -> None:
        while self._work_handles:
            wh = self._work_handles.popleft()
            if wh.handle is not None:
                wh.handle.wait()
            if wh.callback is not None:
                wh.callback()

    def _try_consume_work_handle(self) -> None:
        while self._work_handles and (self._work_handles[0].handle is None or self._work_handles[0].handle.is_completed()):
            wh = self._work_handles.popleft()
            if wh.callback is not None:
                wh.callback()

    def _flush_reduce_calls(self) -> None:
        for bucket in self._bucket_list:
            if not bucket.sent and bucket._params:
                self._send_bucket(bucket)
        self._consume_work_handles()

    def _detect_train_change(self) -> bool:
        with profiler.record_function("fairscale::sdp::detect_train_changes"):
            mask = [_trainable(p) for p in self._all_params]
            changed = mask != self._reference_trainable_mask
            changed |= not self.training and len(self._grad_hooks) > 0
            if self._warn_on_trainable_params_changed and changed:
                logging.warning(
                    "ShardedDDP detected that the trainable params changed, "
                    "either because of eval/train mode or parameter freezing/unfreeze."
                )
            if changed:
                self._reference_trainable_mask = mask
        return changed
