"""Per-layer gradient scaling for fp16 training without a global loss scale.

Capability parity with fairscale/optim/layerwise_gradient_scaler.py:8-289: each named layer can carry its own
scaling factor; full-backward hooks multiply the gradient flowing *into* a layer by its factor and divide the
gradient leaving towards the previous layer, ``unscale`` divides parameter gradients, ``step`` skips the
optimizer when any layer saw inf / nan and grows / backs off the factors.  Layers are taken in
``named_modules()`` order, which has to be the execution order (flat models), as in the reference.  The inf / nan check of a layer is
one multi-tensor sum of squares on CUDA instead of two reductions per parameter.
"""

from __future__ import annotations

from typing import Any, Dict, List, Tuple

import torch
from torch import nn

from ..ops import multi_tensor


class LayerInfo:
    """Book-keeping of one layer: its factor, whether it is scaled at all, growth tracker, overflow flag."""

    def __init__(self, name: str, layer: nn.Module, scale: float = 1.0, scale_layer: bool = False) -> None:
        self.layer_name = name
        self.layer = layer
        self.scaling_factor = scale
        self.found_inf_or_nan = False
        self.growth_tracker = 0
        self.scale_layer = scale_layer


class GradientHelper:
    """Backward hook: scales the gradients w.r.t. the layer inputs by ``inputs_multiplier * outputs_multiplier``
    (undo this layer's factor, apply the previous layer's)."""

    def __init__(self, name: str, inputs_multiplier: float, outputs_multiplier: float):
        self.layer_name = name
        self.inputs_multiplier = inputs_multiplier
        self.outputs_multiplier = outputs_multiplier

    def scale_gradients(self, m: nn.Module, inputs: Tuple, outputs: Tuple) -> Tuple:
        factor = self.inputs_multiplier * self.outputs_multiplier
        return tuple(None if g is None else g * factor for g in inputs)


class LayerwiseGradientScaler:
    def __init__(self, model: nn.Module, layer_scale_dict: Dict[str, float], growth_factor: float = 2.0,
                 backoff_factor: float = 0.5, growth_interval: int = 10000,
                 min_scale: float = torch.finfo(torch.float32).tiny, max_scale: float = torch.finfo(torch.float32).max) -> None:
        self._model = model
        self._layer_scale_dict = layer_scale_dict
        self._growth_factor = growth_factor
        self._backoff_factor = backoff_factor
        self._growth_interval = growth_interval
        self._apply_layerwise_scaling = len(layer_scale_dict) > 0
        self._min_scale = min_scale
        self._max_scale = max_scale
        self._handles: List[Any] = []
        self.layer_info: List[LayerInfo] = []
        if self._apply_layerwise_scaling:
            assert growth_factor > 1.0, "The growth factor must be > 1.0."
            assert backoff_factor < 1.0, "The backoff factor must be < 1.0."
            self.layer_info = [
                LayerInfo(name, layer, layer_scale_dict.get(name, 1.0), name in layer_scale_dict)
                for name, layer in model.named_modules() if name != ""
            ]

    def scale(self) -> None:
        """Install this step's hooks (removed again by :meth:`unscale`)."""
        if not self._apply_layerwise_scaling:
            return
        prev = 1.0
        for info in self.layer_info:
            helper = GradientHelper(info.layer_name, prev, 1.0 / info.scaling_factor)
            self._handles.append(info.layer.register_full_backward_hook(helper.scale_gradients))
            prev = info.scaling_factor
        # The gradient entering the last layer gets that layer's factor, so that the per-layer ratios above
        # telescope and every layer's parameter gradients carry exactly its own factor until unscale().
        last = self.layer_info[-1]
        if last.scaling_factor != 1.0:
            f = last.scaling_factor
            self._handles.append(last.layer.register_full_backward_pre_hook(lambda m, gout: tuple(None if g is None else g * f for g in gout)))

    def unscale(self) -> None:
        if not self._apply_layerwise_scaling:
            return
        for info in self.layer_info:
            if info.found_inf_or_nan:
                continue
            for p in info.layer.parameters():
                if p.grad is not None:
                    p.grad.mul_(1.0 / info.scaling_factor)
        while self._handles:
            self._handles.pop().remove()

    def _check_for_inf_or_nan(self) -> None:
        checks = []
        for info in self.layer_info:
            grads = [p.grad for p in info.layer.parameters() if p.grad is not None]
            info.found_inf_or_nan = False
            if grads:
                if multi_tensor.supported(grads):
                    checks.append((info, multi_tensor.sumsq(grads)))
                else:
                    info.found_inf_or_nan = any(not bool(torch.isfinite(g).all()) for g in grads)
        if checks:  # one device->host read for all layers
            flags = torch.isfinite(torch.cat([c for _, c in checks])).tolist()
            for (info, _), ok in zip(checks, flags):
                info.found_inf_or_nan = not ok

    def step(self, optimizer: Any) -> None:
        if not self._apply_layerwise_scaling:
            optimizer.step()
            return
        self._check_for_inf_or_nan()
        if not any(i.found_inf_or_nan for i in self.layer_info):
            optimizer.step()
        self._update_scale()

    def _clamp(self, v: float) -> float:
        return max(self._min_scale, min(v, self._max_scale))

    def _update_scale(self) -> None:
        for info in self.layer_info:
            if info.found_inf_or_nan:
                if info.scale_layer:
                    info.scaling_factor = self._clamp(self._backoff_factor * info.scaling_factor)
                    info.growth_tracker = 0
            else:
                info.growth_tracker += 1
                if info.scale_layer and info.growth_tracker == self._growth_interval:
                    info.scaling_factor = self._clamp(self._growth_factor * info.scaling_factor)
                    info.growth_tracker = 0

    def get_layer_info(self) -> List[LayerInfo]:
        return self.layer_info

    def get_backward_hooks(self) -> List[Tuple[str, Any]]:
        return [(name, layer._backward_hooks) for name, layer in self._model.named_modules() if name != ""]
