"""state_dict key utilities (interface of fairscale/internal/state_dict.py:16-75)."""

from __future__ import annotations

from typing import TYPE_CHECKING, Dict, Iterator, List, Tuple, Type, Union

from torch import Tensor, nn

if TYPE_CHECKING:
    from collections import OrderedDict


def _walk(module: nn.Module, prefix: str = "") -> Iterator[Tuple[str, nn.Module]]:
    """Depth-first, parents before children, with the state-dict prefix of every module (``""`` for the root, otherwise
    ending in a dot)."""
    yield prefix, module
    for name, child in module.named_children():
        yield from _walk(child, f"{prefix}{name}.")


def find_module_instances(module: nn.Module, search_class: Type[nn.Module]) -> List[Tuple[str, nn.Module]]:
    """``(state_dict_prefix, instance)`` for each ``search_class`` instance under ``module`` (itself included).

    The prefixes are those of the keys the module tree produces once wrapper prefixes have been cleaned, which is what
    state-dict hooks need.
    """
    return [(prefix, m) for prefix, m in _walk(module) if isinstance(m, search_class)]


def replace_by_prefix_(
    state_dict: Union[Dict[str, Tensor], "OrderedDict[str, Tensor]"], old_prefix: str, new_prefix: str
) -> None:
    """Rename, in place, every key starting with ``old_prefix`` to start with ``new_prefix``."""
    if old_prefix == new_prefix:
        raise ValueError("old_prefix and new_prefix must be distinct")
    cut = len(old_prefix)
    for key in [k for k in state_dict if k.startswith(old_prefix)]:
        state_dict[new_prefix + key[cut:]] = state_dict.pop(key)
