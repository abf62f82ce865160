"""Let code and pickles written against ``fairscale`` run on this package.

``install_as_fairscale()`` registers an import hook that resolves ``fairscale`` and every ``fairscale.<sub.module>`` to
the module of the same path under ``fairscale_b200`` (the package mirrors the reference's layout: ``nn.data_parallel``,
``nn.misc.flatten_params_wrapper``, ``optim.oss``, ``experimental.nn.offload`` ...).  After the call

    from fairscale.nn import FullyShardedDataParallel, checkpoint_wrapper
    from fairscale.optim import OSS

import this library, and objects pickled by the reference (for instance a ``FlatParameter`` inside a checkpoint, whose
class path is ``fairscale.nn.misc.flatten_params_wrapper.FlatParameter``) unpickle into the classes defined here.
Nothing is installed unless the function is called, and it refuses to shadow a real ``fairscale`` that is already
imported.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys
from typing import Any, Optional, Sequence

_ALIAS = "fairscale"
_TARGET = "fairscale_b200"


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target_name: str) -> None:
        self.target_name = target_name

    def create_module(self, spec: Any) -> Any:
        return importlib.import_module(self.target_name)  # the very same module object, under a second name

    def exec_module(self, module: Any) -> None:
        pass  # already executed under its own name


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname: str, path: Optional[Sequence[str]] = None, target: Any = None) -> Any:
        if fullname != _ALIAS and not fullname.startswith(_ALIAS + "."):
            return None
        target_name = _TARGET + fullname[len(_ALIAS):]
        try:
            found = importlib.util.find_spec(target_name)
        except (ImportError, ValueError):
            found = None
        if found is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(target_name), is_package=found.submodule_search_locations is not None)
        return spec


_finder: Optional[_AliasFinder] = None


def install_as_fairscale() -> None:
    """Make ``import fairscale...`` resolve to this package (idempotent)."""
    global _finder
    existing = sys.modules.get(_ALIAS)
    if existing is not None and getattr(existing, "__name__", "") != _TARGET:
        raise RuntimeError("a different `fairscale` package is already imported; the alias would shadow it")
    if _finder is None:
        _finder = _AliasFinder()
        sys.meta_path.insert(0, _finder)


def uninstall() -> None:
    """Remove the hook and the aliased entries from ``sys.modules``."""
    global _finder
    if _finder is not None:
        sys.meta_path.remove(_finder)
        _finder = None
    for name in [n for n in sys.modules if n == _ALIAS or n.startswith(_ALIAS + ".")]:
        if getattr(sys.modules[name], "__name__", "").startswith(_TARGET):
            del sys.modules[name]
