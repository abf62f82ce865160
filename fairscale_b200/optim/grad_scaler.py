"""Loss scalers: ``GradScaler`` (accepts fp16 gradients) and the shard-aware ``ShardedGradScaler``.

Capability parity with fairscale/optim/grad_scaler.py:61-415: the sharded scaler agrees on "found inf" across
the ranks that each hold a shard of the gradients (OSS, ShardedDDP, FSDP) and also works for CPU-offloaded
gradients.  What is different on B200:

* the unscale + non-finite check of all gradients of one dtype is one launch of the multi-tensor scale kernel;
* with an optimizer that takes its inverse scale and a skip flag from device memory (``fairscale_b200.optim.Adam``)
  ``step()`` never unscales at all: one multi-tensor sum of squares detects inf / nan, the flag is all-reduced,
  and the fused Adam kernel applies ``1/scale`` while it reads the gradients.  Nothing is read back to the host.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
from torch.amp.grad_scaler import GradScaler as TorchGradScaler
from torch.amp.grad_scaler import OptState

from ..ops import multi_tensor


def _default_device() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


class GradScaler(TorchGradScaler):
    """``torch.amp.GradScaler`` that does not refuse to unscale fp16 gradients (pure-fp16 training)."""

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        if not args and "device" not in kwargs:
            kwargs["device"] = _default_device()
        super().__init__(*args, **kwargs)

    def _unscale_grads_(self, optimizer: Any, inv_scale: torch.Tensor, found_inf: torch.Tensor, allow_fp16: bool) -> Dict[torch.device, torch.Tensor]:
        return super()._unscale_grads_(optimizer, inv_scale, found_inf, True)


class ShardedGradScaler(TorchGradScaler):
    """Args: ``init_scale, growth_factor, backoff_factor, growth_interval, enabled`` as in torch;
    ``process_group``: the ranks whose gradient shards make up one model replica."""

    def __init__(self, init_scale: float = 2.0**16, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True, process_group: Any = None, device: Optional[str] = None) -> None:
        super().__init__(device or _default_device(), init_scale=init_scale, growth_factor=growth_factor,
                         backoff_factor=backoff_factor, growth_interval=growth_interval, enabled=enabled)
        self.group = process_group if process_group is not None else (dist.group.WORLD if dist.is_initialized() else None)

    # ------------------------------------------------------------------ helpers
    def scale(self, outputs: Any) -> Any:
        if not self._enabled:
            return outputs
        if isinstance(outputs, torch.Tensor):
            if self._scale is None:
                self._lazy_init_scale_growth_tracker(outputs.device)
            return outputs * self._scale.to(device=outputs.device, non_blocking=True)  # type: ignore[union-attr]
        if isinstance(outputs, (list, tuple)):
            return type(outputs)(self.scale(o) for o in outputs)
        raise ValueError("outputs must be a Tensor or an iterable of Tensors")

    @staticmethod
    def _grads_by_device(optimizer: Any) -> Dict[torch.device, List[torch.Tensor]]:
        out: Dict[torch.device, List[torch.Tensor]] = defaultdict(list)
        for group in optimizer.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                if g.is_sparse:
                    g = g.coalesce()._values() if g.dtype is torch.float16 else g._values()
                out[g.device].append(g)
        return out

    def _all_reduce_found_inf(self, found: Dict[torch.device, torch.Tensor]) -> None:
        if self.group is None or not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return
        works = []
        for dev, t in found.items():
            if dev.type == "cpu" and dist.get_backend(self.group) == "nccl":
                t_dev = t.cuda()
                dist.all_reduce(t_dev, group=self.group)
                t.copy_(t_dev)
            else:
                works.append(dist.all_reduce(t, group=self.group, async_op=True))
        for w in works:
            w.wait()

    # ------------------------------------------------------------------ torch hooks
    @torch.no_grad()
    def _unscale_grads_(self, optimizer: Any, inv_scale: torch.Tensor, found_inf: torch.Tensor, allow_fp16: bool = True) -> Dict[torch.device, torch.Tensor]:
        result: Dict[torch.device, torch.Tensor] = {}
        for dev, grads in self._grads_by_device(optimizer).items():
            inv = inv_scale.to(dev, non_blocking=True)
            if dev.type == "cuda" and multi_tensor.supported(grads):
                flag = torch.zeros(1, dtype=torch.int32, device=dev)
                multi_tensor.scale_(grads, inv.reshape(1), flag)
                result[dev] = flag.to(torch.float32).reshape(())
            else:
                f = found_inf.to(dev, copy=True)
                by_dtype: Dict[torch.dtype, List[torch.Tensor]] = defaultdict(list)
                for g in grads:
                    by_dtype[g.dtype].append(g)
                for gs in by_dtype.values():
                    try:
                        torch._amp_foreach_non_finite_check_and_unscale_(gs, f, inv)
                    except (RuntimeError, NotImplementedError):
                        for g in gs:
                            if not bool(torch.isfinite(g).all()):
                                f.fill_(1.0)
                            g.mul_(inv.to(g.dtype))
                result[dev] = f
        if not result:  # a rank whose shard holds no parameter still takes part in the agreement
            result[found_inf.device] = found_inf.clone()
        return result

    def unscale_(self, optimizer: Any) -> None:
        if not self._enabled:
            return
        super().unscale_(optimizer)
        self._all_reduce_found_inf(self._per_optimizer_states[id(optimizer)]["found_inf_per_device"])

    def _fusable(self, optimizer: Any) -> bool:
        return hasattr(optimizer, "noop_flag") and hasattr(optimizer, "inv_scale") and self._scale is not None and self._scale.is_cuda

    def step(self, optimizer: Any, *args: Any, **kwargs: Any) -> Optional[float]:
        if not self._enabled:
            return optimizer.step(*args, **kwargs)
        state = self._per_optimizer_states[id(optimizer)]
        if state["stage"] is OptState.READY and self._fusable(optimizer) and "closure" not in kwargs:
            self._check_scale_growth_tracker("step")
            grads = self._grads_by_device(optimizer)
            if len(grads) == 1 and multi_tensor.supported(next(iter(grads.values()))):
                (dev, gs), = grads.items()
                found = (~torch.isfinite(multi_tensor.sumsq(gs))).to(torch.float32).reshape(())
                per_dev = {dev: found}
                self._all_reduce_found_inf(per_dev)
                state["found_inf_per_device"] = per_dev
                prev = (optimizer.noop_flag, optimizer.inv_scale)
                optimizer.noop_flag = (found > 0).to(torch.int32).reshape(1)
                optimizer.inv_scale = self._scale.to(dev).double().reciprocal().float().reshape(1)  # type: ignore[union-attr]
                try:
                    ret = optimizer.step(*args, **kwargs)
                finally:
                    optimizer.noop_flag, optimizer.inv_scale = prev
                state["stage"] = OptState.STEPPED
                return ret
        if state["stage"] is OptState.READY:
            self.unscale_(optimizer)
        return super().step(optimizer, *args, **kwargs)
