"""Per-tensor-parallel-rank random streams and an RNG-aware activation checkpoint.

Parity: fairscale/nn/model_parallel/random.py:39-250.  Two streams exist on every rank: the default
one (equal inside a model-parallel group, for dropout on replicated activations) and the tracked
"model-parallel-rng" one (seed + 2718 + tp_rank, for dropout on sharded activations and weight init).
The tracker works on CPU-only hosts too (it then forks the CPU generator), which keeps the CPU test tier
meaningful.
"""

from __future__ import annotations

import contextlib
from typing import Any, Dict, Iterator, Set, Union

import torch
import torch.distributed as dist
from torch.utils.checkpoint import detach_variable

from .initialize import get_data_parallel_rank, get_model_parallel_rank

__all__ = [
    "checkpoint",
    "get_cuda_rng_tracker",
    "model_parallel_cuda_manual_seed",
]


_MODEL_PARALLEL_RNG_TRACKER_NAME = "model-parallel-rng"


def _has_cuda() -> bool:
    return torch.cuda.is_available()


def _get_state() -> torch.Tensor:
    return torch.cuda.get_rng_state() if _has_cuda() else torch.get_rng_state()


def _set_cuda_rng_state(new_state: torch.Tensor, device: Union[int, str, torch.device] = -1) -> None:
    """Install ``new_state`` without cloning it (cloning per fork is measurable with many GPUs)."""
    if not _has_cuda():
        torch.set_rng_state(new_state)
        return
    if device == -1:
        dev = torch.device("cuda")
    elif isinstance(device, str):
        dev = torch.device(device)
    elif isinstance(device, int):
        dev = torch.device("cuda", device)
    else:
        dev = device

    def apply() -> None:
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        torch.cuda.default_generators[idx].set_state(new_state)

    torch.cuda._lazy_call(apply)


def _seed(seed: int) -> None:
    if _has_cuda():
        torch.cuda.manual_seed(seed)
    else:
        torch.manual_seed(seed)


class CudaRNGStatesTracker:
    """Named RNG states that can be temporarily made current with :meth:`fork`."""

    def __init__(self) -> None:
        self.states_: Dict[str, torch.Tensor] = {}
        self.seeds_: Set[int] = set()

    def reset(self) -> None:
        self.states_ = {}
        self.seeds_ = set()

    def get_states(self) -> Dict[str, torch.Tensor]:
        return dict(self.states_)

    def set_states(self, states: Dict[str, torch.Tensor]) -> None:
        self.states_ = states

    def add(self, name: str, seed: int) -> None:
        if seed in self.seeds_:
            raise Exception(f"seed {seed} already exists")
        self.seeds_.add(seed)
        if name in self.states_:
            raise Exception(f"cuda rng state {name} already exists")
        saved = _get_state()
        _seed(seed)
        self.states_[name] = _get_state()
        _set_cuda_rng_state(saved)

    @contextlib.contextmanager
    def fork(self, name: str = _MODEL_PARALLEL_RNG_TRACKER_NAME) -> Iterator[None]:
        if name not in self.states_:
            raise Exception(f"cuda rng state {name} is not added")
        saved = _get_state()
        _set_cuda_rng_state(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = _get_state()
            _set_cuda_rng_state(saved)


_CUDA_RNG_STATE_TRACKER = CudaRNGStatesTracker()


def get_cuda_rng_tracker() -> CudaRNGStatesTracker:
    return _CUDA_RNG_STATE_TRACKER


def model_parallel_cuda_manual_seed(seed: int) -> None:
    """Seed both streams; call after ``initialize_model_parallel`` and instead of ``torch.cuda.manual_seed``."""
    mp_seed = seed + 2718 + get_model_parallel_rank()
    if dist.get_rank() == 0:
        print(
            f"> initializing model parallel cuda seeds on global rank {dist.get_rank()}, model parallel rank "
            f"{get_model_parallel_rank()}, and data parallel rank {get_data_parallel_rank()} with model parallel seed: "
            f"{mp_seed} and data parallel seed: {seed}",
            flush=True,
        )
    _CUDA_RNG_STATE_TRACKER.reset()
    _seed(seed)
    _CUDA_RNG_STATE_TRACKER.add(_MODEL_PARALLEL_RNG_TRACKER_NAME, mp_seed)


class CheckpointFunction(torch.autograd.Function):
    """``torch.utils.checkpoint`` that also saves / restores the tracked model-parallel RNG states."""

    @staticmethod
    def forward(ctx: Any, run_function: Any, *args: Any) -> Any:  # type: ignore[override]
        ctx.run_function = run_function
        ctx.fwd_cpu_rng_state = torch.get_rng_state()
        ctx.fwd_dev_rng_state = _get_state()
        ctx.fwd_tracker = get_cuda_rng_tracker().get_states()
        ctx.autocast = next(({"device_type": d, "dtype": torch.get_autocast_dtype(d)} for d in ("cuda", "cpu") if torch.is_autocast_enabled(d)), None)
        ctx.save_for_backward(*args)
        with torch.no_grad():
            return run_function(*args)

    @staticmethod
    def backward(ctx: Any, *grads: Any) -> Any:  # type: ignore[override]
        if not torch.autograd._is_checkpoint_valid():
            raise RuntimeError("Checkpointing is not compatible with .grad(), please use .backward() if possible")
        inputs = ctx.saved_tensors
        now_cpu, now_dev, now_tracker = torch.get_rng_state(), _get_state(), get_cuda_rng_tracker().get_states()
        torch.set_rng_state(ctx.fwd_cpu_rng_state)
        _set_cuda_rng_state(ctx.fwd_dev_rng_state)
        get_cuda_rng_tracker().set_states(ctx.fwd_tracker)
        detached = detach_variable(inputs)
        amp = torch.autocast(**ctx.autocast) if ctx.autocast is not None else contextlib.nullcontext()
        with torch.enable_grad(), amp:  # the forward's autocast state, as well as its random states
            outputs = ctx.run_function(*detached)
        torch.set_rng_state(now_cpu)
        _set_cuda_rng_state(now_dev)
        get_cuda_rng_tracker().set_states(now_tracker)
        if isinstance(outputs, torch.Tensor):
            outputs = (outputs,)
        torch.autograd.backward(outputs, grads)
        return (None,) + tuple(t.grad for t in detached)


def checkpoint(function: Any, *args: Any) -> Any:
    """Run ``function(*args)`` without storing activations; recompute (with identical dropout) in backward."""
    return CheckpointFunction.apply(function, *args)
