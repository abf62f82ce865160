"""Helpers for tests about memory (parity: fairscale/fair_dev/testing/testing_memory.py:14-37)."""

import gc
from typing import Tuple

import torch


def find_tensor_by_shape(target_shape: Tuple, only_param: bool = True) -> bool:
    """True when a live tensor (by default: a live ``nn.Parameter``) of exactly ``target_shape`` exists; used to
    check that something was or was not freed."""
    for obj in gc.get_objects():
        try:
            if only_param and not isinstance(obj, torch.nn.Parameter):
                continue
            if torch.is_tensor(obj) and tuple(obj.shape) == tuple(target_shape):
                return True
        except Exception:
            continue
    return False
