"""AdaScale: learning-rate gain from the ratio of gradient variance to gradient norm at large batch sizes.

Capability parity with fairscale/optim/adascale.py:49-726 (``AdaScale`` wrapping any optimizer, gradient
accumulation, per-param-group gain, debiased / plain EWMA, ``AdaScaleWrapper`` with an optimizer-like
constructor).  The statistics are the paper's (appendix B.3):

    var  = (S / (cN - 1)) * (mean_i |g_i|^2 - |g|^2)        sqr = |g|^2 - var / S        gain = (var + sqr) / (var / S + sqr)

with ``g_i`` the cN per-rank, per-accumulation-pass gradients, ``g`` their mean and ``S`` the scale.
Per-pass squared norms are accumulated on the device inside tensor hooks; the squared norm of the averaged
gradient is one multi-tensor sum of squares per param group, and a step reads back one small tensor instead of
one ``.item()`` per parameter.
"""

from __future__ import annotations

import functools
from typing import Any, Dict, List, Optional, Type

import numpy as np
import torch
import torch.distributed as dist
from torch.autograd import Variable
from torch.optim import SGD, Optimizer

from ..ops import multi_tensor


class AdaScale(Optimizer):
    def __init__(self, optimizer: Optimizer, world_size: Optional[int] = None, scale: Optional[float] = None,
                 smoothing: Optional[float] = None, num_gradients_to_accumulate: int = 1, is_scaled_loss: bool = True,
                 debias_ewma: bool = True):
        self._hook_handles: List[Any] = []
        self._optimizer = optimizer
        self._local_grad_sqr: Optional[torch.Tensor] = None
        self._world_size = world_size if world_size is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        self._num_backward_calls = 0
        self._last_final_backward_call = 0
        self._debias_ewma = debias_ewma
        self._is_scaled_loss = is_scaled_loss
        self._final_callback_queued = False
        self.param_groups = optimizer.param_groups  # lr schedulers act on the wrapped optimizer's groups
        self.set_num_gradients_to_accumulate(num_gradients_to_accumulate, update_smoothing=True)
        if smoothing is not None:
            self._smoothing = smoothing
        if self._world_size * self._num_grads_to_accum <= 1:
            raise RuntimeError("AdaScale does not support a single worker without grad accumulation.")
        n = len(optimizer.param_groups)
        optimizer.state.setdefault("adascale", {"grad_sqr_avg": np.ones(n), "grad_var_avg": np.zeros(n)})
        self.set_scale(self._world_size * self._num_grads_to_accum if scale is None else scale)
        self._hook()

    # ------------------------------------------------------------------ hooks
    def _hook(self) -> None:
        assert self._hook_handles == [], "Must run unhook first"
        for idx, group in enumerate(self._optimizer.param_groups):
            for p in group["params"]:
                self._hook_handles.append(p.register_hook(functools.partial(self._backward_hook, idx)))

    def unhook(self) -> None:
        """Remove the tensor hooks (they keep parameters alive); also needed before the object can be collected."""
        for h in self._hook_handles:
            h.remove()
        self._hook_handles = []

    def __del__(self) -> None:
        self.unhook()

    # ------------------------------------------------------------------ properties
    @property
    def _state(self) -> Dict[str, np.ndarray]:
        return self._optimizer.state["adascale"]

    @property
    def scale(self) -> float:
        """Batch-size scaling factor relative to the baseline run (not the gain)."""
        return self._scale

    @property
    def smoothing(self) -> float:
        return self._smoothing

    def set_scale(self, scale: float, update_estimate: bool = True) -> None:
        assert self._local_grad_sqr is None, "Don't change scale in backward phase"
        assert scale >= 1, "Scale must be at least 1"
        if update_estimate and hasattr(self, "_scale"):
            ratio = self._scale / scale  # variance of the mean gradient shrinks with the batch
            for key in ("grad_var_avg_biased" if self._debias_ewma else "grad_var_avg_total", "grad_var_avg"):
                if key in self._state:
                    self._state[key] = self._state[key] * ratio
        self._scale = scale

    def _grad_sqr_avg(self, pg_idx: Optional[int] = None) -> float:
        v = self._state["grad_sqr_avg"]
        return float(v[pg_idx]) if pg_idx is not None else float(np.sum(v))

    def _grad_var_avg(self, pg_idx: Optional[int] = None) -> float:
        v = self._state["grad_var_avg"]
        return float(v[pg_idx]) if pg_idx is not None else float(np.sum(v))

    def gain(self, pg_idx: Optional[int] = None) -> float:
        """Current gain ratio r_t, in [1, scale]; for one param group or over all of them."""
        var, sqr = self._grad_var_avg(pg_idx), self._grad_sqr_avg(pg_idx)
        return (var + sqr) / (var / self.scale + sqr)

    # ------------------------------------------------------------------ statistics
    def _update_avg(self, name: str, value: np.ndarray, factor: float) -> None:
        st = self._state
        if self._debias_ewma:
            biased = factor * st.get(name + "_biased", np.zeros(value.shape[0])) + (1.0 - factor) * value
            unbias = factor * st.get(name + "_unbias", np.zeros(value.shape[0])) + (1.0 - factor)
            st[name + "_biased"], st[name + "_unbias"], st[name] = biased, unbias, biased / unbias
            return
        count = st.get(name + "_count", np.zeros(1))
        count[0] += 1
        st[name + "_count"] = count
        if count < 1 / (1 - self._smoothing):  # plain mean until the window is full
            total = st.get(name + "_total")
            total = value.copy() if total is None else total + value
            st[name + "_total"] = total
            st[name] = total / count
        else:
            st[name] = factor * st[name] + (1.0 - factor) * value

    def _gather_flat_grad(self) -> torch.Tensor:
        views = []
        for group in self._optimizer.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    views.append(p.new_zeros(p.numel()))
                else:
                    views.append((p.grad.to_dense() if p.grad.is_sparse else p.grad).reshape(-1))
        return torch.cat(views, 0)

    def _compute_intra_grad_corr_mean(self) -> torch.Tensor:
        """Mean pairwise correlation of the ranks' local gradients (call under ``no_sync``)."""
        assert self._world_size > 1, "Only for distributed training"
        flat = self._gather_flat_grad()
        gathered = [torch.zeros_like(flat) for _ in range(self._world_size)]
        dist.all_gather(gathered, flat)
        corr = torch.stack(gathered).float().corrcoef()
        return corr[torch.triu(torch.ones_like(corr), diagonal=1) == 1].mean()

    def _backward_hook(self, pg_idx: int, grad: torch.Tensor) -> None:
        if self._local_grad_sqr is None:
            self._local_grad_sqr = torch.zeros(len(self._optimizer.param_groups), device=grad.device, dtype=torch.float32)
        self._local_grad_sqr[pg_idx] += grad.detach().float().pow(2).sum()
        # run the final step after every other end-of-backward callback (DDP's gradient averaging included):
        # a callback that queues the real callback.
        self._final_callback_queued = False
        Variable._execution_engine.queue_callback(self._queue_callback)

    def _queue_callback(self) -> None:
        if self._final_callback_queued:
            return
        self._final_callback_queued = True
        Variable._execution_engine.queue_callback(self._final_callback)

    def _total_grad_sqr(self) -> np.ndarray:
        sums = []
        for group in self._optimizer.param_groups:
            grads = [p.grad.detach() for p in group["params"] if p.grad is not None]
            if grads and multi_tensor.supported(grads):
                sums.append(multi_tensor.sumsq(grads).reshape(()))
            elif grads:
                sums.append(torch.stack([g.float().pow(2).sum() for g in grads]).sum())
            else:
                sums.append(torch.zeros((), device=self._local_grad_sqr.device))  # type: ignore[union-attr]
        return torch.stack([s.to(sums[0].device) for s in sums]).double().cpu().numpy()

    def _final_callback(self) -> None:
        self._final_callback_queued = False
        assert isinstance(self._local_grad_sqr, torch.Tensor)
        self._num_backward_calls += 1
        done = self._num_backward_calls - self._last_final_backward_call
        assert done <= self._num_grads_to_accum, f"bug: {done} backward passes for {self._num_grads_to_accum} to accumulate"
        if done % self._num_grads_to_accum != 0:
            return  # still accumulating
        work = dist.all_reduce(self._local_grad_sqr, async_op=True) if self._world_size > 1 else None
        total_grad_sqr = self._total_grad_sqr()
        if work is not None:
            work.wait()
        local_grad_sqr = self._local_grad_sqr.double().cpu().numpy()
        if self._num_grads_to_accum > 1:
            # bring per-pass norms and the accumulated gradient's norm to the same loss scale
            if self._is_scaled_loss:
                local_grad_sqr = local_grad_sqr * self._num_grads_to_accum**2
            else:
                total_grad_sqr = total_grad_sqr / self._num_grads_to_accum**2
        S, cN = self._scale, self._world_size * self._num_grads_to_accum
        grad_var = local_grad_sqr * (S / cN) / (cN - 1) - total_grad_sqr * S / (cN - 1)
        grad_sqr = total_grad_sqr - grad_var / S
        self._update_avg("grad_sqr_avg", np.maximum(grad_sqr, 0.0), self.smoothing)
        self._update_avg("grad_var_avg", np.maximum(grad_var, 1e-6), self.smoothing)
        self._last_final_backward_call = self._num_backward_calls
        self._local_grad_sqr = None

    # ------------------------------------------------------------------ optimizer protocol
    def step(self, *args: Any, **kwargs: Any) -> Optional[float]:
        """``optimizer.step`` with every group's lr multiplied by that group's gain for this one step."""
        assert self._local_grad_sqr is None, "Don't step without finishing backward phase"
        saved = [g["lr"] for g in self._optimizer.param_groups]
        for idx, g in enumerate(self._optimizer.param_groups):
            g["lr"] = g["lr"] * self.gain(pg_idx=idx)
        try:
            return self._optimizer.step(*args, **kwargs)
        finally:
            for lr, g in zip(saved, self._optimizer.param_groups):
                g["lr"] = lr

    def add_param_group(self, pg: Dict) -> None:
        assert self._local_grad_sqr is None, "Can't add parameter group during backward"
        self._optimizer.add_param_group(pg)
        self.unhook()
        self._hook()
        for name in list(self._state.keys()):
            assert name.startswith("grad_sqr_avg") or name.startswith("grad_var_avg"), name
            if name.endswith("_count"):
                continue
            self._state[name] = np.append(self._state[name], 1 if name == "grad_sqr_avg" else 0)
            assert self._state[name].shape == (len(self._optimizer.param_groups),)

    def zero_grad(self, *args: Any, **kwargs: Any) -> None:  # type: ignore[override]
        assert self._local_grad_sqr is None, "Don't zero_grad in backward"
        return self._optimizer.zero_grad(*args, **kwargs)

    def state_dict(self) -> Dict:
        """The wrapped optimizer's state (do not checkpoint in the middle of an accumulation window)."""
        assert self._local_grad_sqr is None, "Don't checkpoint in backward"
        return self._optimizer.state_dict()

    def load_state_dict(self, data: Dict) -> None:
        assert self._local_grad_sqr is None, "Don't load checkpoint in backward"
        return self._optimizer.load_state_dict(data)

    def set_num_gradients_to_accumulate(self, num_gradients_to_accumulate: int, update_smoothing: bool = True) -> None:
        assert self._local_grad_sqr is None, "Don't change num_grad_to_accum in backward"
        assert num_gradients_to_accumulate >= 1, f"Invalid value {num_gradients_to_accumulate}"
        self._num_grads_to_accum = num_gradients_to_accumulate
        if update_smoothing:
            self._smoothing = max(1 - self._world_size * self._num_grads_to_accum / 1000, 0)

    def scale_grad_by_num_grads_to_accum(self) -> None:
        """After accumulating with an unscaled loss, divide the gradients by the number of passes."""
        assert self._local_grad_sqr is None, "Only call this after backward"
        assert self._num_grads_to_accum > 1, "Must be accumulating gradients"
        assert not self._is_scaled_loss, "Must use unscaled loss"
        for group in self._optimizer.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    p.grad.div_(self._num_grads_to_accum)

    def __getattr__(self, name: str) -> Any:
        """Anything else (``state``, ``defaults``, extension methods) is the wrapped optimizer's."""
        opt = self.__dict__.get("_optimizer")
        if opt is None or name.startswith("__"):
            raise AttributeError(name)
        return getattr(opt, name)


class AdaScaleWrapper(AdaScale):
    """AdaScale with an optimizer-style constructor (``params`` first) so it can sit under wrappers like OSS."""

    def __init__(self, params: Any, world_size: Optional[int] = None, scale: Optional[float] = None,
                 smoothing: Optional[float] = None, num_gradients_to_accumulate: int = 1, debias_ewma: bool = True,
                 optim_cls: Type[Optimizer] = SGD, **additional_optim_args: Any):
        super().__init__(optim_cls(params, **additional_optim_args), world_size, scale, smoothing,
                         num_gradients_to_accumulate, True, debias_ewma)
