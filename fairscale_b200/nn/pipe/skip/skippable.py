"""The ``@skippable`` decorator and its ``stash`` / ``pop`` commands.

API parity with fairscale/nn/pipe/skip/skippable.py:52-453.  A skippable module's ``forward`` is a generator:
``yield stash(name, tensor)`` parks a tensor, ``tensor = yield pop(name)`` retrieves one parked by an earlier
layer; the tensor travels outside the sequential data flow (and, under ``Pipe``, outside the autograd graph
through portals) to the partition that pops it.
"""

from __future__ import annotations

from typing import (
    Any,
    Callable,
    ClassVar,
    Dict,
    FrozenSet,
    Generator,
    Iterable,
    List,
    Optional,
    Set,
    Tuple,
    Type,
    TypeVar,
    Union,
    cast,
)

from torch import Tensor, nn

from ..microbatch import Batch
from .namespace import Namespace
from .tracker import current_skip_tracker

__all__ = ["skippable", "stash", "pop", "verify_skippables"]

Tensors = Tuple[Tensor, ...]
TensorOrTensors = Union[Tensor, Tensors]
T = TypeVar("T", bound="Skippable")


class Skippable(nn.Module):
    """Base of the classes produced by :func:`skippable`; do not subclass directly."""

    module_cls: ClassVar[Type[nn.Module]]
    stashable_names: ClassVar[FrozenSet[str]]
    poppable_names: ClassVar[FrozenSet[str]]

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__()
        self.module = self.module_cls(*args, **kwargs)
        self.namespaces: Dict[str, Namespace] = {}

    def __repr__(self) -> str:
        return f"@skippable({self.module})"

    def namespaced(self, name: str) -> Tuple[Namespace, str]:
        return (cast(Namespace, self.namespaces.get(name)), name)

    def stashable(self) -> Iterable[Tuple[Namespace, str]]:
        for name in self.stashable_names:
            yield self.namespaced(name)

    def poppable(self) -> Iterable[Tuple[Namespace, str]]:
        for name in self.poppable_names:
            yield self.namespaced(name)

    def isolate(self: T, ns: Namespace, *, only: Optional[Iterable[str]] = None) -> T:
        """Put all (or ``only`` the listed) skip names of this layer into namespace ``ns`` so the same
        names can be reused by another stash/pop pair in the same sequential model."""
        names: Iterable[str] = self.stashable_names | self.poppable_names if only is None else set(only)
        for name in names:
            self.namespaces[name] = ns
        return self

    def dispatch(self, input: Any, handle_stash: Callable[[str, Optional[Tensor]], None], handle_pop: Callable[[str], Optional[Tensor]]) -> Any:
        """Drive the generator returned by the wrapped module's ``forward``."""
        gen = self.module(input)
        if not isinstance(gen, Generator):
            return gen  # an ordinary forward
        try:
            op = next(gen)
            while True:
                if isinstance(op, stash):
                    handle_stash(op.name, op.tensor)
                    op = next(gen)
                elif isinstance(op, pop):
                    op = gen.send(handle_pop(op.name))
                else:
                    raise TypeError(f"{op!r} is not a command from @skippable")
        except StopIteration as stop:
            return stop.args[0]

    def forward(self, input: TensorOrTensors) -> TensorOrTensors:  # type: ignore[override]
        """Skip tensors to pop are fetched *before* the wrapped module runs (the fetch forks the graph from the
        input) and stashed tensors are filed *after* it (the filing joins into the output); that ordering is
        what lets portals keep backward correct under ``Pipe``."""
        tracker = current_skip_tracker()
        stashed: Dict[str, Optional[Tensor]] = {}
        poppable: Dict[str, Optional[Tensor]] = {}

        batch = Batch(input, tracker.index)
        for ns, name in self.poppable():
            try:
                poppable[name] = tracker.load(batch, ns, name)
            except KeyError:
                raise RuntimeError(f"'{name}' has not been stashed")
        input = batch.tensor_or_tensors

        def on_stash(name: str, tensor: Optional[Tensor]) -> None:
            if name not in self.stashable_names:
                raise RuntimeError(f"'{name}' has not been declared as stashable")
            stashed[name] = tensor

        def on_pop(name: str) -> Optional[Tensor]:
            if name not in self.poppable_names:
                raise RuntimeError(f"'{name}' has not been declared as poppable")
            return poppable.pop(name)

        output = self.dispatch(input, on_stash, on_pop)

        missing_stash = self.stashable_names - stashed.keys()
        if missing_stash:
            raise RuntimeError(f"{', '.join(repr(n) for n in sorted(missing_stash))} must be stashed but have not")
        if poppable:
            raise RuntimeError(f"{', '.join(repr(n) for n in sorted(poppable))} must be popped but have not")

        batch = Batch(output, tracker.index)
        for ns, name in self.stashable():
            tracker.save(batch, ns, name, stashed[name])
        return batch.tensor_or_tensors


def skippable(stash: Iterable[str] = (), pop: Iterable[str] = ()) -> Callable[[Type[nn.Module]], Type[Skippable]]:
    """Class decorator declaring which skip names a module stashes and pops::

        @skippable(stash=["skip"])
        class Stash(nn.Module):
            def forward(self, x):
                yield stash("skip", x)
                return x
    """
    stashable_names = frozenset(stash)
    poppable_names = frozenset(pop)

    def extend(module_cls: Type[nn.Module]) -> Type[Skippable]:
        name = module_cls.__name__
        bases = (Skippable,)
        attrs = {"module_cls": module_cls, "stashable_names": stashable_names, "poppable_names": poppable_names}
        return type(name, bases, attrs)

    return extend


class stash:
    """``yield stash(name, tensor)`` inside a skippable forward."""

    __slots__ = ("name", "tensor")

    def __init__(self, name: str, tensor: Optional[Tensor]) -> None:
        self.name = name
        self.tensor = tensor


class pop:
    """``tensor = yield pop(name)`` inside a skippable forward."""

    __slots__ = ("name",)

    def __init__(self, name: str) -> None:
        self.name = name


def verify_skippables(module: nn.Sequential) -> None:
    """Check that every stash has exactly one later pop in the same namespace (and vice versa).

    Raises ``TypeError`` listing every violation: pop before stash, stash never popped, a name declared
    twice by different layers, or one layer that both stashes and pops the same name.
    """
    stashed: Set[Tuple[Namespace, str]] = set()
    popped: Set[Tuple[Namespace, str]] = set()
    msgs: List[str] = []
    for layer_name, layer in module.named_children():
        if not isinstance(layer, Skippable):
            continue
        for name in layer.stashable_names & layer.poppable_names:
            msgs.append(f"'{layer_name}' declared '{name}' both as stashable and as poppable")
        for ns, name in layer.stashable():
            if name in layer.poppable_names:
                continue
            if (ns, name) in stashed:
                msgs.append(f"'{layer_name}' redeclared '{name}' as stashable but not isolated by namespace")
                continue
            stashed.add((ns, name))
        for ns, name in layer.poppable():
            if name in layer.stashable_names:
                continue
            if (ns, name) in popped:
                msgs.append(f"'{layer_name}' redeclared '{name}' as poppable but not isolated by namespace")
                continue
            if (ns, name) not in stashed:
                msgs.append(f"'{layer_name}' declared '{name}' as poppable but it was not stashed")
                continue
            popped.add((ns, name))
    for _, name in stashed - popped:
        msgs.append(f"no module declared '{name}' as poppable but stashed")
    if msgs:
        raise TypeError("one or more pairs of stash and pop do not match:\n\n%s" % "\n".join("* %s" % x for x in msgs))
