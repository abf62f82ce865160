"""fairseq-style dynamic loss scaler that also works on CPU tensors.

Same behaviour and public names as fairscale/experimental/optim/dynamic_loss_scaler.py:32-208, organised as two parts: a
small schedule object that only counts steps and decides when the scale moves (it never sees a tensor), and the scaler
proper that measures gradient norms, drives the schedule and talks to the optimizer.

Rules of the schedule: a step whose gradient norm is inf or nan is an overflow.  Overflows are counted since the last
change of the scale; once their share of the steps since then reaches ``tolerance`` the scale is divided by
``scale_factor`` (not below ``threshold``).  After ``scale_window`` steps without overflow the scale is multiplied by
``scale_factor``.  A scale that would reach ``min_loss_scale`` stops training with ``FloatingPointError``.

On CUDA the norm of a parameter group's gradients is one multi-tensor launch and one host read, not one norm per tensor.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional

import torch

from ...ops import multi_tensor


class OptState(Enum):
    READY = 0
    UNSCALED = 1
    STEPPED = 2


@dataclass
class _Schedule:
    """Step counters of the scaler.  ``step`` counts calls of ``update`` (and overflowing steps), the other two remember at
    which step the scale last changed and last overflowed."""

    window: int
    tolerance: float
    step: int = 0
    last_overflow: int = -1
    last_change: int = -1
    overflows_since_change: int = 0

    def overflow_forces_decrease(self) -> bool:
        """Register an overflow at the current step; True when the tolerated share is used up."""
        self.last_overflow = self.step
        self.overflows_since_change += 1
        share = self.overflows_since_change / float(self.step - self.last_change)
        if share < self.tolerance:
            return False
        self.last_change, self.overflows_since_change = self.step, 0
        return True

    def clean_step_allows_increase(self) -> bool:
        """Called once per finished step: True every ``window`` steps after the last overflow."""
        grow = (self.step - self.last_overflow) % self.window == 0
        if grow:
            self.last_change = self.step
        self.step += 1
        return grow


@dataclass
class _PerOptimizer:
    stage: Dict[int, OptState] = field(default_factory=dict)

    def of(self, optimizer: Any) -> OptState:
        return self.stage.get(id(optimizer), OptState.READY)

    def set(self, optimizer: Any, value: OptState) -> None:
        self.stage[id(optimizer)] = value


class DynamicLossScaler:
    def __init__(self, init_scale: float = 2.0**15, scale_factor: float = 2.0, scale_window: int = 2000,
                 tolerance: float = 0.0, threshold: Optional[float] = None, min_loss_scale: float = 1e-4):
        self.loss_scale = init_scale
        self.scale_factor = scale_factor
        self.scale_window = scale_window
        self.tolerance = tolerance
        self.threshold = threshold
        self.min_loss_scale = min_loss_scale
        self._schedule = _Schedule(window=scale_window, tolerance=tolerance)
        self._optimizers = _PerOptimizer()

    # ------------------------------------------------------------------ scaling
    def scale(self, outputs: Any) -> Any:
        """``outputs`` (a tensor, or a list / tuple of tensors) times the current scale."""
        if isinstance(outputs, (list, tuple)):
            return type(outputs)(o * self.loss_scale for o in outputs)
        return outputs * self.loss_scale

    @torch.no_grad()
    def unscale_(self, optimizer: Any) -> None:
        stage = self._optimizers.of(optimizer)
        if stage is OptState.UNSCALED:
            raise RuntimeError("unscale_() has already been called on this optimizer since the last update().")
        if stage is OptState.STEPPED:
            raise RuntimeError("unscale_() is being called after step().")
        grads = [p.grad for group in optimizer.param_groups for p in group["params"] if p.grad is not None]
        if grads:
            torch._foreach_mul_(grads, 1.0 / float(self.loss_scale))
        self._optimizers.set(optimizer, OptState.UNSCALED)

    # ------------------------------------------------------------------ overflow handling
    @torch.no_grad()
    def _get_gradients_norm(self, params: List[torch.nn.Parameter]) -> float:
        grads = [p.grad.detach() for p in params if p.grad is not None]
        if not grads:
            return 0.0
        if multi_tensor.supported(grads):
            return float(multi_tensor.l2_norm(grads))
        per_tensor = torch.stack([torch.linalg.vector_norm(g.float()) for g in grads])
        return float(torch.linalg.vector_norm(per_tensor))

    def _decrease_loss_scale(self) -> None:
        lowered = self.loss_scale / self.scale_factor
        self.loss_scale = lowered if self.threshold is None else max(lowered, self.threshold)

    def _check_overflow(self, grad_norm: float) -> None:
        """Raises ``OverflowError`` (after adjusting the scale) when ``grad_norm`` is not finite."""
        if math.isfinite(grad_norm):
            return
        before = self.loss_scale
        if self._schedule.overflow_forces_decrease():
            self._decrease_loss_scale()
        if self.loss_scale <= self.min_loss_scale:
            self.loss_scale = before  # leave the scale usable for whoever catches the error
            raise FloatingPointError(
                f"Minimum loss scale reached ({self.min_loss_scale}). Your loss is probably exploding. Try lowering the "
                "learning rate, using gradient clipping or increasing the batch size."
            )
        self._schedule.step += 1
        raise OverflowError("setting loss scale to: " + str(self.loss_scale))

    # ------------------------------------------------------------------ the training-loop calls
    def step(self, optimizer: Any, *args: Any, **kwargs: Any) -> Any:
        """Unscale (if not done yet) and step; returns None and skips the step when the gradients overflowed."""
        if "closure" in kwargs:
            raise RuntimeError("Closure use is not currently supported if DynamicLossScaler is enabled.")
        if self._optimizers.of(optimizer) is OptState.STEPPED:
            raise RuntimeError("step() has already been called since the last update().")
        try:
            for group in optimizer.param_groups:
                self._check_overflow(self._get_gradients_norm(group["params"]))
        except OverflowError:
            return None
        if self._optimizers.of(optimizer) is OptState.READY:
            self.unscale_(optimizer)
        result = optimizer.step(*args, **kwargs)
        self._optimizers.set(optimizer, OptState.STEPPED)
        return result

    def update(self) -> None:
        """End of a step: grow the scale when the window without overflow is complete, forget per-optimizer stages."""
        if self._schedule.clean_step_allows_increase():
            self.loss_scale *= self.scale_factor
        self._optimizers.stage.clear()

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> Optional[Dict[str, float]]:
        return None if self.loss_scale is None else {"loss_scale": self.loss_scale}

    def load_state_dict(self, state_dict: Dict[str, float]) -> None:
        self.loss_scale = state_dict.get("loss_scale", self.loss_scale)
