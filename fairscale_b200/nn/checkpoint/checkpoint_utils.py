"""BatchNorm guard for activation checkpointing (parity: fairscale/nn/checkpoint/checkpoint_utils.py:13-50)."""

from __future__ import annotations

from typing import Any, List

import torch
from torch import nn
from torch.nn.modules.batchnorm import _BatchNorm


def _suspend_tracking(bn: _BatchNorm, _inputs: Any) -> None:
    if not torch.is_grad_enabled():
        bn._track_running_stats_backup = bn.track_running_stats  # type: ignore[assignment]
        bn.track_running_stats = False


def _resume_tracking(bn: _BatchNorm, _inputs: Any, _result: Any) -> None:
    if not torch.is_grad_enabled():
        bn.track_running_stats = bn._track_running_stats_backup  # type: ignore[assignment]


def patch_batchnorm(module: nn.Module) -> List:
    """Stop every BatchNorm under ``module`` from updating running statistics while grad is disabled.

    A checkpointed block runs forward twice (once without grad, once recomputing); only the
    recomputation may touch the statistics or they would be updated twice per step.  A layer
    carrying a ``disable_patch_batchnorm`` attribute is left alone.  Returns the hook handles.
    """
    handles: List[Any] = []
    for child in module.modules():
        if isinstance(child, _BatchNorm) and not hasattr(child, "disable_patch_batchnorm"):
            handles.append(child.register_forward_pre_hook(_suspend_tracking))
            handles.append(child.register_forward_hook(_resume_tracking))
    return handles
