"""Context-driven (recursive) wrapping of sub-modules.

API parity with fairscale/nn/wrap/auto_wrap.py:12-331: ``enable_wrap`` establishes a
wrapper class and default kwargs; ``wrap`` applies it to a module (no-op outside the
context); ``auto_wrap`` walks a module bottom-up and wraps every sub-tree a policy
approves.  The active configuration lives in a small context object rather than in
class attributes.
"""

from __future__ import annotations

import contextlib
from typing import Any, Callable, Dict, Generator, Optional, Set, Tuple, Type, cast

import torch.nn as nn


def default_auto_wrap_policy(
    module: nn.Module,
    recurse: bool,
    unwrapped_params: int,
    module_is_root: bool,
    min_num_params: int = int(1e8),
    force_leaf_modules: Optional[Set[Type[nn.Module]]] = None,
    exclude_wrap_modules: Optional[Set[Type[nn.Module]]] = None,
    skip_params_check_for_root: bool = False,
) -> bool:
    """Size-based policy.

    Called twice per module: with ``recurse=True`` to decide whether to descend into
    its children, with ``recurse=False`` to decide whether to wrap the module itself
    given ``unwrapped_params`` parameters not yet claimed by wrapped children.  A custom
    policy must accept the first four arguments.
    """
    leaves = default_auto_wrap_policy.FORCE_LEAF_MODULES if force_leaf_modules is None else force_leaf_modules  # type: ignore[attr-defined]
    excluded = default_auto_wrap_policy.EXCLUDE_WRAP_MODULES if exclude_wrap_modules is None else exclude_wrap_modules  # type: ignore[attr-defined]
    big_enough = unwrapped_params >= min_num_params
    if recurse:
        return big_enough and not isinstance(module, tuple(leaves))
    wanted = big_enough or (module_is_root and skip_params_check_for_root)
    return wanted and not isinstance(module, tuple(excluded))


# containers have no forward of their own; MultiheadAttention accesses its children's weights directly
default_auto_wrap_policy.EXCLUDE_WRAP_MODULES = {nn.ModuleList, nn.ModuleDict}  # type: ignore[attr-defined]
default_auto_wrap_policy.FORCE_LEAF_MODULES = {nn.MultiheadAttention}  # type: ignore[attr-defined]


def config_auto_wrap_policy(module: nn.Module, recurse: bool, unwrapped_params: int, module_is_root: bool) -> bool:
    """Wrap exactly the modules tagged with a ``wrapper_config`` attribute; always descend."""
    return True if recurse else hasattr(module, "wrapper_config")


class ConfigAutoWrap:
    """State of the active ``enable_wrap`` context (class-level, so ``wrap`` can find it)."""

    in_autowrap_context: bool = False
    move_module_cuda_half: bool = False
    wrapper_cls: Optional[Callable] = None
    kwargs: Dict[str, Any] = {}
    auto_wrap_policy: Optional[Callable] = None

    def __init__(self, auto_wrap_policy: Optional[Callable] = None, **kwargs: Any):
        self.auto_wrap_policy = auto_wrap_policy
        self.kwargs = kwargs

    @staticmethod
    def enable_autowrap_context(auto_wrap_policy: Optional[Callable], kwargs: Any) -> None:
        if ConfigAutoWrap.in_autowrap_context:
            raise NotImplementedError(
                "You are already within an autowrap context and we currently do not supported nested autowrap."
            )
        kwargs = dict(kwargs)
        assert "wrapper_cls" in kwargs
        ConfigAutoWrap.in_autowrap_context = True
        ConfigAutoWrap.move_module_cuda_half = bool(kwargs.pop("move_module_cuda_half", False))
        ConfigAutoWrap.wrapper_cls = cast(Callable, kwargs.pop("wrapper_cls"))
        ConfigAutoWrap.auto_wrap_policy = default_auto_wrap_policy if auto_wrap_policy is None else auto_wrap_policy
        ConfigAutoWrap.kwargs = kwargs

    @staticmethod
    def disable_autowrap_context() -> None:
        ConfigAutoWrap.in_autowrap_context = False
        ConfigAutoWrap.move_module_cuda_half = False
        ConfigAutoWrap.wrapper_cls = None
        ConfigAutoWrap.kwargs = {}
        ConfigAutoWrap.auto_wrap_policy = None

    def __enter__(self) -> None:
        self.enable_autowrap_context(self.auto_wrap_policy, self.kwargs)

    def __exit__(self, exc_type: Any, exc_val: Any, exc_tb: Any) -> None:
        self.disable_autowrap_context()

    @staticmethod
    def recursive_wrap(
        module: nn.Module, auto_wrap_policy: Optional[Callable], module_is_root: bool, **kwargs: Any
    ) -> Tuple[nn.Module, int]:
        """Post-order walk; returns ``(possibly wrapped module, number of parameters now under a wrapper)``."""
        policy = ConfigAutoWrap.auto_wrap_policy if auto_wrap_policy is None else auto_wrap_policy
        assert policy is not None
        wrapper_type = cast(type, ConfigAutoWrap.wrapper_cls)
        for _, sub in module.named_modules():
            assert not isinstance(sub, wrapper_type), "auto_wrap found an already wrapped sub-module"

        total = sum(p.numel() for p in module.parameters())
        if not policy(module=module, recurse=True, unwrapped_params=total, module_is_root=module_is_root):
            return module, 0
        claimed = 0
        for name, child in module.named_children():
            new_child, n = ConfigAutoWrap.recursive_wrap(
                module=child, auto_wrap_policy=policy, module_is_root=False, **kwargs
            )
            setattr(module, name, new_child)
            claimed += n
        if policy(module=module, recurse=False, unwrapped_params=total - claimed, module_is_root=module_is_root):
            return wrap(module, **kwargs), total
        return module, claimed


@contextlib.contextmanager
def enable_wrap(auto_wrap_policy: Optional[Callable] = None, **wrapper_kwargs: Any) -> Generator[None, None, None]:
    """Inside this context ``wrap``/``auto_wrap`` apply ``wrapper_cls(module, **wrapper_kwargs)``.

    Wrapping layer by layer at construction shards big layers immediately, so the
    unsharded model never has to fit in memory.  Required kwarg: ``wrapper_cls``;
    optional ``move_module_cuda_half`` moves each module to CUDA fp16 before wrapping.
    """
    with ConfigAutoWrap(auto_wrap_policy, **wrapper_kwargs):
        yield


def wrap(module: nn.Module, **wrap_overrides: Any) -> nn.Module:
    """Wrap ``module`` if an ``enable_wrap`` context is active, else return it unchanged.

    kwargs precedence (low → high): context defaults, ``module.wrapper_config``, ``wrap_overrides``.
    """
    if not ConfigAutoWrap.in_autowrap_context:
        return module
    per_module: Dict[str, Any] = {}
    if hasattr(module, "wrapper_config"):
        per_module = module.wrapper_config  # type: ignore[assignment]
        assert isinstance(per_module, dict)
    merged = {**ConfigAutoWrap.kwargs, **per_module, **wrap_overrides}
    assert ConfigAutoWrap.wrapper_cls is not None
    if ConfigAutoWrap.move_module_cuda_half:
        module = module.cuda().half()
    return ConfigAutoWrap.wrapper_cls(module, **merged)


def auto_wrap(module: nn.Module, auto_wrap_policy: Optional[Callable] = None, **kwargs: Any) -> nn.Module:
    """Recursively wrap the sub-modules of ``module`` approved by the policy (once per module tree).

    Shared parameters must end up under the same wrapper or the sharing is lost.
    """
    if not ConfigAutoWrap.in_autowrap_context:
        return module
    wrapped, _ = ConfigAutoWrap.recursive_wrap(module, auto_wrap_policy=auto_wrap_policy, module_is_root=True, **kwargs)
    return wrapped
