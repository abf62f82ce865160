"""state_dict key utilities (parity: fairscale/internal/state_dict.py:16-75)."""

from __future__ import annotations

from typing import TYPE_CHECKING, Dict, List, Tuple, Type, Union

import torch
from torch import Tensor, nn

if TYPE_CHECKING:
    from collections import OrderedDict


def find_module_instances(module: nn.Module, search_class: Type[nn.Module]) -> List[Tuple[str, nn.Module]]:
    """Return ``(state_dict_prefix, instance)`` for each ``search_class`` instance under ``module``.

    Prefixes end with ``"."`` (or are empty for the root) and follow the key names the
    module tree produces *after* wrapper prefixes were cleaned, which is what
    state-dict hooks need.
    """
    found: List[Tuple[str, nn.Module]] = []

    def visit(mod: nn.Module, prefix: str) -> None:
        if isinstance(mod, search_class):
            found.append((prefix, mod))
        for name, child in mod.named_children():
            visit(child, f"{prefix}{name}.")

    visit(module, "")
    return found


def replace_by_prefix_(
    state_dict: Union[Dict[str, Tensor], "OrderedDict[str, Tensor]"], old_prefix: str, new_prefix: str
) -> None:
    """Rename, in place, every key starting with ``old_prefix`` to start with ``new_prefix``."""
    if old_prefix == new_prefix:
        raise ValueError("old_prefix and new_prefix must be distinct")
    for key in list(state_dict.keys()):
        if key.startswith(old_prefix):
            state_dict[new_prefix + key[len(old_prefix):]] = state_dict.pop(key)
