"""``@skippable`` modules: layers that hand a tensor to a later layer around the sequential data flow.

    @skippable(stash=["residual"])
    class Save(nn.Module):
        def forward(self, x):
            yield stash("residual", x)
            return self.conv(x)

    @skippable(pop=["residual"])
    class Add(nn.Module):
        def forward(self, x):
            residual = yield pop("residual")
            return x + residual

The wrapped ``forward`` is a generator that yields :class:`stash` / :class:`pop` commands; the wrapper executes them
against the current skip tracker (``skip/tracker.py``).  User-facing behaviour and error messages follow
fairscale/nn/pipe/skip/skippable.py:52-453.
"""

from __future__ import annotations

import inspect
from typing import Any, Callable, ClassVar, Dict, FrozenSet, Iterable, Iterator, List, Optional, Tuple, Type, TypeVar, Union

from torch import Tensor, nn

from ..microbatch import Batch
from .layout import SkipKey
from .namespace import Namespace
from .tracker import current_skip_tracker

__all__ = ["skippable", "stash", "pop", "verify_skippables"]

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]
S = TypeVar("S", bound="Skippable")


class stash:
    """Command: ``yield stash(name, tensor)`` files ``tensor`` (or None) under ``name``."""

    __slots__ = ("name", "tensor")

    def __init__(self, name: str, tensor: Optional[Tensor]) -> None:
        self.name, self.tensor = name, tensor


class pop:
    """Command: ``tensor = yield pop(name)`` fetches what an earlier layer stashed under ``name``."""

    __slots__ = ("name",)

    def __init__(self, name: str) -> None:
        self.name = name


def _quoted(names: Iterable[str]) -> str:
    return ", ".join(f"'{n}'" for n in sorted(names))


class Skippable(nn.Module):
    """What :func:`skippable` makes of a module class.  Holds an instance of the original class as ``self.module``."""

    module_cls: ClassVar[Type[nn.Module]]
    stashable_names: ClassVar[FrozenSet[str]]
    poppable_names: ClassVar[FrozenSet[str]]

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__()
        self.module = self.module_cls(*args, **kwargs)
        self.namespaces: Dict[str, Namespace] = {}

    def __repr__(self) -> str:
        return f"@skippable({self.module})"

    # -- names and namespaces
    def namespaced(self, name: str) -> SkipKey:
        return (self.namespaces.get(name), name)

    def stashable(self) -> Iterator[SkipKey]:
        return (self.namespaced(n) for n in self.stashable_names)

    def poppable(self) -> Iterator[SkipKey]:
        return (self.namespaced(n) for n in self.poppable_names)

    def isolate(self: S, ns: Namespace, *, only: Optional[Iterable[str]] = None) -> S:
        """Move this layer's skip names (all of them, or ``only`` the given ones) into namespace ``ns``; returns self."""
        for name in (self.stashable_names | self.poppable_names) if only is None else only:
            self.namespaces[name] = ns
        return self

    # -- running the generator
    def dispatch(self, input: Any, handle_stash: Callable[[str, Optional[Tensor]], None],
                 handle_pop: Callable[[str], Optional[Tensor]]) -> Any:
        """Call the wrapped module; if its forward is a generator, serve its commands until it returns."""
        running = self.module(input)
        if not inspect.isgenerator(running):
            return running
        reply: Optional[Tensor] = None
        while True:
            try:
                command = running.send(reply)
            except StopIteration as finished:
                return finished.value
            if isinstance(command, stash):
                handle_stash(command.name, command.tensor)
                reply = None
            elif isinstance(command, pop):
                reply = handle_pop(command.name)
            else:
                raise TypeError(f"{command!r} is not a command from @skippable")

    def forward(self, input: TensorOrTensors) -> TensorOrTensors:  # type: ignore[override]
        tracker = current_skip_tracker()
        carrier = Batch(input, tracker.index)

        # everything this layer may pop is fetched up front, everything it stashes is filed after it has run
        fetched: Dict[str, Optional[Tensor]] = {}
        for ns, name in self.poppable():
            try:
                fetched[name] = tracker.load(carrier, ns, name)
            except KeyError:
                raise RuntimeError(f"'{name}' has not been stashed") from None
        filed: Dict[str, Optional[Tensor]] = {}

        def on_stash(name: str, tensor: Optional[Tensor]) -> None:
            if name not in self.stashable_names:
                raise RuntimeError(f"'{name}' has not been declared as stashable")
            filed[name] = tensor

        def on_pop(name: str) -> Optional[Tensor]:
            if name not in self.poppable_names:
                raise RuntimeError(f"'{name}' has not been declared as poppable")
            return fetched.pop(name)

        output = self.dispatch(carrier.tensor_or_tensors, on_stash, on_pop)

        unstashed = self.stashable_names - filed.keys()
        if unstashed:
            raise RuntimeError(f"{_quoted(unstashed)} must be stashed but have not")
        if fetched:
            raise RuntimeError(f"{_quoted(fetched)} must be popped but have not")

        carrier = Batch(output, tracker.index)
        for ns, name in self.stashable():
            tracker.save(carrier, ns, name, filed[name])
        return carrier.tensor_or_tensors


def skippable(stash: Iterable[str] = (), pop: Iterable[str] = ()) -> Callable[[Type[nn.Module]], Type[Skippable]]:
    """Class decorator: declares the names the module may stash and pop and wraps it into a :class:`Skippable`."""
    declared = {"stashable_names": frozenset(stash), "poppable_names": frozenset(pop)}

    def wrap(module_cls: Type[nn.Module]) -> Type[Skippable]:
        return type(module_cls.__name__, (Skippable,), dict(declared, module_cls=module_cls))

    return wrap


def verify_skippables(module: nn.Sequential) -> None:
    """``TypeError`` listing every stash / pop mismatch of ``module``: a pop without an earlier stash, a stash nobody
    pops, a name two layers declare in the same namespace, a layer that declares one name both ways."""
    open_stashes: Dict[SkipKey, str] = {}  # stashed and not yet popped -> layer that stashed
    closed: set = set()
    problems: List[str] = []
    for layer_name, layer in module.named_children():
        if not isinstance(layer, Skippable):
            continue
        both = layer.stashable_names & layer.poppable_names
        for name in sorted(both):
            problems.append(f"'{layer_name}' declared '{name}' both as stashable and as poppable")
        for key in layer.stashable():
            if key[1] in both:
                continue
            if key in open_stashes or key in closed:
                problems.append(f"'{layer_name}' redeclared '{key[1]}' as stashable but not isolated by namespace")
            else:
                open_stashes[key] = layer_name
        for key in layer.poppable():
            if key[1] in both:
                continue
            if key in closed:
                problems.append(f"'{layer_name}' redeclared '{key[1]}' as poppable but not isolated by namespace")
            elif key not in open_stashes:
                problems.append(f"'{layer_name}' declared '{key[1]}' as poppable but it was not stashed")
            else:
                del open_stashes[key]
                closed.add(key)
    for (_, name) in open_stashes:
        problems.append(f"no module declared '{name}' as poppable but stashed")
    if problems:
        raise TypeError("one or more pairs of stash and pop do not match:\n\n" + "\n".join(f"* {p}" for p in problems))
