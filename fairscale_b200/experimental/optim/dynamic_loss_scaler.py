"""fairseq-style dynamic loss scaler that also works on CPU tensors.

Capability parity with fairscale/experimental/optim/dynamic_loss_scaler.py:32-208: overflow is detected through
the gradient norm (inf / nan), the scale shrinks by ``scale_factor`` when the share of overflowing steps since
the last rescale reaches ``tolerance``, grows every ``scale_window`` overflow-free steps, and training stops
with ``FloatingPointError`` once the scale would fall to ``min_loss_scale``.  On CUDA the norm of all gradients
is one multi-tensor launch and one host read per step, not one ``torch.norm`` per parameter.
"""

from __future__ import annotations

from collections import defaultdict
from enum import Enum
from typing import Any, Dict, List, Optional

import torch

from ...ops import multi_tensor


class OptState(Enum):
    READY = 0
    UNSCALED = 1
    STEPPED = 2


class DynamicLossScaler:
    def __init__(self, init_scale: float = 2.0**15, scale_factor: float = 2.0, scale_window: int = 2000,
                 tolerance: float = 0.0, threshold: Optional[float] = None, min_loss_scale: float = 1e-4):
        self.loss_scale = init_scale
        self.scale_factor = scale_factor
        self.scale_window = scale_window
        self.tolerance = tolerance
        self.threshold = threshold
        self.min_loss_scale = min_loss_scale
        self._iter = 0
        self._last_overflow_iter = -1
        self._last_rescale_iter = -1
        self._overflows_since_rescale = 0
        self._stage: Dict[int, OptState] = defaultdict(lambda: OptState.READY)

    def scale(self, outputs: Any) -> Any:
        if isinstance(outputs, (list, tuple)):
            return type(outputs)(self.loss_scale * o for o in outputs)
        return self.loss_scale * outputs

    @torch.no_grad()
    def _get_gradients_norm(self, params: List[torch.nn.Parameter]) -> float:
        grads = [p.grad.detach() for p in params if p.grad is not None]
        if not grads:
            return 0.0
        if multi_tensor.supported(grads):
            return float(multi_tensor.l2_norm(grads))
        return float(torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(g.float()) for g in grads])))

    def _decrease_loss_scale(self) -> None:
        self.loss_scale /= self.scale_factor
        if self.threshold is not None:
            self.loss_scale = max(self.loss_scale, self.threshold)

    def _check_overflow(self, grad_norm: float) -> None:
        if grad_norm != float("inf") and grad_norm == grad_norm:
            return
        prev = self.loss_scale
        since = self._iter - self._last_rescale_iter
        self._last_overflow_iter = self._iter
        self._overflows_since_rescale += 1
        if self._overflows_since_rescale / float(since) >= self.tolerance:
            self._decrease_loss_scale()
            self._last_rescale_iter = self._iter
            self._overflows_since_rescale = 0
        if self.loss_scale <= self.min_loss_scale:
            self.loss_scale = prev
            raise FloatingPointError(
                f"Minimum loss scale reached ({self.min_loss_scale}). Your loss is probably exploding. Try lowering the "
                "learning rate, using gradient clipping or increasing the batch size."
            )
        self._iter += 1
        raise OverflowError("setting loss scale to: " + str(self.loss_scale))

    def update(self) -> None:
        if (self._iter - self._last_overflow_iter) % self.scale_window == 0:
            self.loss_scale *= self.scale_factor
            self._last_rescale_iter = self._iter
        self._iter += 1
        self._stage.clear()

    def step(self, optimizer: Any, *args: Any, **kwargs: Any) -> Any:
        """Unscale (if not done yet) and step; returns None and skips the step when the gradients overflowed."""
        if "closure" in kwargs:
            raise RuntimeError("Closure use is not currently supported if DynamicLossScaler is enabled.")
        if self._stage[id(optimizer)] is OptState.STEPPED:
            raise RuntimeError("step() has already been called since the last update().")
        for group in optimizer.param_groups:
            try:
                self._check_overflow(self._get_gradients_norm(group["params"]))
            except OverflowError:
                return None
        if self._stage[id(optimizer)] is OptState.READY:
            self.unscale_(optimizer)
        ret = optimizer.step(*args, **kwargs)
        self._stage[id(optimizer)] = OptState.STEPPED
        return ret

    @torch.no_grad()
    def unscale_(self, optimizer: Any) -> None:
        stage = self._stage[id(optimizer)]
        if stage is OptState.UNSCALED:
            raise RuntimeError("unscale_() has already been called on this optimizer since the last update().")
        if stage is OptState.STEPPED:
            raise RuntimeError("unscale_() is being called after step().")
        inv = 1.0 / float(self.loss_scale)
        for group in optimizer.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    p.grad.mul_(inv)
        self._stage[id(optimizer)] = OptState.UNSCALED

    def state_dict(self) -> Optional[Dict[str, float]]:
        return {"loss_scale": self.loss_scale} if self.loss_scale is not None else None

    def load_state_dict(self, state_dict: Dict[str, float]) -> None:
        if "loss_scale" in state_dict:
            self.loss_scale = state_dict["loss_scale"]
