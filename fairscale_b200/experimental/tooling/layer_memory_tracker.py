"""Layer-by-layer memory tracing of forward and backward, with FSDP all-gather volume and checkpoint suggestions.

Capability parity with fairscale/experimental/tooling/layer_memory_tracker.py:59-782: module hooks record the
allocator state and the size of freshly allocated activations around every module, traces can be saved / loaded
as JSON, ``find_best_reset_points`` / ``suggest_checkpoint_location`` place activation checkpoints to minimise
the peak, and the traces can be plotted when matplotlib is installed.

All-gather traffic is observed through a listener on this library's communication front-end, which also sees
the NVLink kernels that never touch a ``ProcessGroup``; :class:`ProcessGroupTracker` remains as a thin marker
that restricts the accounting to one group.  Device synchronisation per hook makes tracing slow by design.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum, auto
from functools import lru_cache
import json
from typing import Any, Callable, Dict, List, NamedTuple, Optional, Set, Tuple, Union

from contextlib import contextmanager

import torch
from torch import nn

from ...parallel import comm


@dataclass
class TraceForwardEvent:
    """memory_diff: allocator delta over the module's forward; memory_activations: bytes of new output tensors."""

    memory_diff: int
    memory_activations: int

    def to_dict(self) -> Dict[str, Any]:
        return {"memory_diff": self.memory_diff, "memory_activations": self.memory_activations}

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TraceForwardEvent":
        return cls(memory_diff=d["memory_diff"], memory_activations=d["memory_activations"])


@dataclass
class TraceBackwardEvent:
    memory_activations: int

    def to_dict(self) -> Dict[str, Any]:
        return {"memory_activations": self.memory_activations}

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TraceBackwardEvent":
        return cls(memory_activations=d["memory_activations"])


class LayerMemoryTrace(NamedTuple):
    module_name: str
    module_params: int
    allocated: int
    reserved: int
    is_forward: bool
    all_gathered: int
    cumul_all_gathered: int
    event: Union[TraceForwardEvent, TraceBackwardEvent]

    def to_dict(self) -> Dict[str, Any]:
        d = self._asdict()
        d["event"] = self.event.to_dict()
        return d

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LayerMemoryTrace":
        ev_cls = TraceForwardEvent if d["is_forward"] else TraceBackwardEvent
        return cls(**{**d, "event": ev_cls.from_dict(d["event"])})


@dataclass
class LayerwiseMemoryTrackerSummary:
    max_memory_allocated: int
    max_memory_cached: int
    total_activation_allocations: int
    total_forward_allocations: int
    top_forward_activation_producers: List[LayerMemoryTrace]


class ProcessGroupTrackingEvent(Enum):
    allgather = auto()


class ProcessGroupTracker:
    """Marks ``group`` as the one whose all-gathers a tracker should count; every other attribute is the group's."""

    def __init__(self, group: Any, listener: Optional[Callable] = None):
        self.group = group
        self.listener = listener

    def __getattr__(self, item: str) -> Any:
        return getattr(self.group, item)


def _nbytes(xs: Any) -> int:
    if isinstance(xs, torch.Tensor):
        return xs.numel() * xs.element_size()
    if isinstance(xs, (tuple, list)):
        return sum(_nbytes(x) for x in xs)
    return 0


def _tensors(xs: Any) -> List[torch.Tensor]:
    out: List[torch.Tensor] = []
    stack = [xs]
    while stack:
        x = stack.pop()
        if isinstance(x, torch.Tensor):
            out.append(x)
        elif isinstance(x, (tuple, list)):
            stack.extend(x)
        elif isinstance(x, dict):
            stack.extend(x.values())
    return out


class LayerwiseMemoryTracker:
    def __init__(self) -> None:
        self.memory_traces: List[LayerMemoryTrace] = []
        self._hooks: List[Any] = []
        self._previous_module_name: Optional[str] = None
        self._last_all_gather_memory = 0
        self._cumul_all_gather_memory: List[int] = []
        self._memory_pre_forward = 0
        self._traced_module_names: Set[str] = set()
        self._groups: Optional[Set[int]] = None
        self._listening = False

    # ------------------------------------------------------------------ control
    def monitor(self, model: nn.Module) -> None:
        """Install the hooks.  FSDP instances found in ``model`` have their all-gathers accounted."""
        from ...nn.data_parallel import FullyShardedDataParallel

        for name, m in model.named_modules():
            self._hooks.append(m.register_forward_pre_hook(self._pre_forward(name)))
            self._hooks.append(m.register_forward_hook(self._post_forward(name)))
            self._hooks.append(m.register_full_backward_hook(self._backward(name)))
            if isinstance(m, FullyShardedDataParallel) and isinstance(m.process_group, ProcessGroupTracker):
                self._groups = (self._groups or set()) | {id(m.process_group), id(m.process_group.group)}
        comm.add_listener(self._on_collective)
        self._listening = True
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def clear_traces(self) -> None:
        self.memory_traces.clear()

    def stop(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        if self._listening:
            comm.remove_listener(self._on_collective)
            self._listening = False
        self._previous_module_name = None
        self._memory_pre_forward = 0
        self._last_all_gather_memory = 0
        self._cumul_all_gather_memory.clear()

    # ------------------------------------------------------------------ views
    @property
    def forward_traces(self) -> List[LayerMemoryTrace]:
        return [t for t in self.memory_traces if t.is_forward]

    @property
    def backward_traces(self) -> List[LayerMemoryTrace]:
        return [t for t in self.memory_traces if not t.is_forward]

    @property
    def max_memory_allocated(self) -> int:
        return max(t.allocated for t in self.memory_traces)

    @property
    def max_memory_cached(self) -> int:
        return max(t.reserved for t in self.memory_traces)

    def top_forward_activation_producers(self, top: int = 10) -> List[LayerMemoryTrace]:
        return sorted(self.forward_traces, key=lambda t: t.event.memory_activations, reverse=True)[:top]

    @property
    def summary(self) -> LayerwiseMemoryTrackerSummary:
        return LayerwiseMemoryTrackerSummary(
            max_memory_allocated=self.max_memory_allocated,
            max_memory_cached=self.max_memory_cached,
            total_activation_allocations=sum(t.event.memory_activations for t in self.forward_traces),
            total_forward_allocations=sum(t.event.memory_diff for t in self.forward_traces),  # type: ignore[union-attr]
            top_forward_activation_producers=self.top_forward_activation_producers(10),
        )

    def show_plots(self, figsize: Tuple[int, int] = (16, 20), capture: bool = False) -> Optional[Any]:
        return compare_memory_traces_in_plot({"run": self.memory_traces}, figsize=figsize, capture=capture)

    def save_traces(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"traces": [t.to_dict() for t in self.memory_traces]}, f)

    @classmethod
    def load(cls, path: str) -> "LayerwiseMemoryTracker":
        out = cls()
        with open(path) as f:
            out.memory_traces = [LayerMemoryTrace.from_dict(t) for t in json.load(f)["traces"]]
        return out

    # ------------------------------------------------------------------ hooks
    @staticmethod
    def _capture_memory() -> Tuple[int, int]:
        if not torch.cuda.is_available():
            return 0, 0
        torch.cuda.synchronize()
        return torch.cuda.memory_allocated(), torch.cuda.memory_reserved()

    @staticmethod
    def _get_parameter_size(module: nn.Module) -> int:
        return sum(p.numel() * p.element_size() for p in module.parameters())

    @staticmethod
    def _filter_allocated_output(inputs: Any, outputs: Any) -> List[torch.Tensor]:
        """Outputs that own fresh storage (not views of an input)."""
        seen = {x.untyped_storage().data_ptr() for x in _tensors(inputs)}
        return [y for y in _tensors(outputs) if y.untyped_storage().data_ptr() not in seen]

    def _is_fsdp(self, module: nn.Module) -> bool:
        from ...nn.data_parallel import FullyShardedDataParallel

        return isinstance(module, FullyShardedDataParallel)

    def _on_collective(self, kind: str, group: Any, out: Any, inp: Any) -> None:
        if kind != "all_gather" or (self._groups is not None and id(group) not in self._groups):
            return
        size = _nbytes(out)
        self._last_all_gather_memory += size
        if self._cumul_all_gather_memory:
            self._cumul_all_gather_memory[-1] += size

    def _pre_forward(self, name: str) -> Callable:
        def hook(module: nn.Module, inputs: Any) -> None:
            allocated, _ = self._capture_memory()
            self._previous_module_name = name
            self._memory_pre_forward = allocated
            if self._is_fsdp(module):
                self._cumul_all_gather_memory.append(0)

        return hook

    def _post_forward(self, name: str) -> Callable:
        def hook(module: nn.Module, inputs: Any, outputs: Any) -> None:
            if self._is_fsdp(module) and self._cumul_all_gather_memory:
                self._cumul_all_gather_memory.pop()
            if name == self._previous_module_name:  # a leaf in the hook sense: nothing ran in between
                allocated, reserved = self._capture_memory()
                self._traced_module_names.add(name)
                acts = sum(_nbytes(y) for y in self._filter_allocated_output(inputs, outputs))
                self.memory_traces.append(LayerMemoryTrace(
                    module_name=name, module_params=self._get_parameter_size(module), allocated=allocated, reserved=reserved,
                    is_forward=True, all_gathered=self._last_all_gather_memory,
                    cumul_all_gathered=sum(self._cumul_all_gather_memory),
                    event=TraceForwardEvent(memory_diff=allocated - self._memory_pre_forward, memory_activations=acts)))
                self._last_all_gather_memory = 0
            self._previous_module_name = None
            self._memory_pre_forward = 0

        return hook

    def _backward(self, name: str) -> Callable:
        def hook(module: nn.Module, grad_input: Any, grad_output: Any) -> None:
            if name not in self._traced_module_names:
                return
            mem = sum(_nbytes(y) for y in self._filter_allocated_output(grad_input, grad_output))
            allocated, reserved = self._capture_memory()
            self.memory_traces.append(LayerMemoryTrace(
                module_name=name, module_params=self._get_parameter_size(module), allocated=allocated, reserved=reserved,
                is_forward=False, all_gathered=self._last_all_gather_memory, cumul_all_gathered=0,
                event=TraceBackwardEvent(memory_activations=mem)))
            self._last_all_gather_memory = 0

        return hook


def find_best_reset_points(activation_sizes: List[int], num_checkpoints: int) -> Tuple[int, List[int]]:
    """Split the layer sequence into ``num_checkpoints + 1`` consecutive segments minimising the largest segment
    sum (the activation peak when memory is reset at every boundary).  Returns (peak, boundary indices)."""
    n = len(activation_sizes)
    prefix = [0]
    for a in activation_sizes:
        prefix.append(prefix[-1] + a)

    @lru_cache(maxsize=None)
    def best(pos: int, remaining: int) -> Tuple[int, Tuple[int, ...]]:
        if pos == n:
            return 0, ()
        if remaining == 0:
            return prefix[n] - prefix[pos], ()
        top: Tuple[int, Tuple[int, ...]] = (1 << 62, ())
        for cut in range(pos + 1, n + 1):
            rest, cuts = best(cut, remaining - 1)
            score = max(prefix[cut] - prefix[pos], rest)
            if score < top[0]:
                top = (score, (cut,) + cuts)
        return top

    score, cuts = best(0, num_checkpoints)
    return int(score), list(cuts)


@dataclass
class SuggestedCheckpoints:
    max_memory: int
    split_modules: List[str]
    all_modules: List[str]


def suggest_checkpoint_location(traces: List[LayerMemoryTrace], num_checkpoints: int, num_skipped_layers: int = 0) -> SuggestedCheckpoints:
    """Names of the modules at which to start a new ``checkpoint_wrapper`` segment."""
    modules: List[str] = []
    sizes: List[int] = []
    for t in traces:
        if t.is_forward and t.module_name not in modules:
            modules.append(t.module_name)
            sizes.append(t.event.memory_activations)
    modules, sizes = modules[num_skipped_layers:], sizes[num_skipped_layers:]
    peak, cuts = find_best_reset_points(sizes, num_checkpoints)
    return SuggestedCheckpoints(max_memory=peak, split_modules=[modules[i] for i in cuts if i < len(modules)], all_modules=modules)


def compare_memory_traces_in_plot(memory_traces_by_job: Dict[str, List[LayerMemoryTrace]], figsize: Tuple[int, int] = (16, 20),
                                  capture: bool = False) -> Optional[Any]:
    """Plot allocated / reserved memory, activation sizes, parameter sizes and all-gather volumes per run."""
    try:
        import matplotlib.pyplot as plt
    except ImportError as e:  # pragma: no cover
        raise ImportError("plotting memory traces needs matplotlib (`pip install matplotlib`)") from e
    fig, ax = plt.subplots(figsize=figsize, ncols=2, nrows=3)
    gb = 2**30
    for job, traces in memory_traces_by_job.items():
        fwd = [t for t in traces if t.is_forward]
        ax[0, 0].plot([t.allocated / gb for t in traces], label=job)
        ax[0, 1].plot([t.reserved / gb for t in traces], label=job)
        ax[1, 0].plot([t.event.memory_activations / gb for t in fwd], label=job)
        ax[1, 1].plot([t.module_params / gb for t in fwd], label=job)
        ax[2, 0].plot([t.all_gathered / gb for t in traces], label=job)
        ax[2, 1].plot([t.cumul_all_gathered / gb for t in traces], label=job)
    for a, title in zip(ax.flat, ["allocated (GB)", "reserved (GB)", "forward activations (GB)", "parameters (GB)",
                                 "all-gathered (GB)", "cumulative all-gathered (GB)"]):
        a.set_title(title)
        a.legend()
    if not capture:
        plt.show()
        return None
    import io

    buf = io.BytesIO()
    fig.savefig(buf, format="png")
    plt.close(fig)
    return buf.getvalue()


@contextmanager
def null_context() -> Iterator[None]:
    yield


def matplotlib_figure_to_image(fig: Any) -> Any:
    """Render a matplotlib figure to an RGB ``PIL.Image`` (for saving a plot of the traces)."""
    import io

    from PIL import Image

    buf = io.BytesIO()
    fig.savefig(buf)
    buf.seek(0)
    return Image.open(buf).convert("RGB")
