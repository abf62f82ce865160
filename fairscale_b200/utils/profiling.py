"""Tracing helpers: named ranges that show up both in the PyTorch profiler and (as NVTX) in Nsight, CUDA-event
timers, a Chrome-trace exporter and a sampler of SM clocks / throttle reasons.

The range names are the ones the reference emits through ``record_function`` (``fairscale::oss::optim_step``,
``fairscale::sdp::forward``, ``chunk%d-part%d``, ``fairscale.experimental.nn.offload:*`` ...; see
fairscale/optim/oss.py:223-592, fairscale/nn/data_parallel/sharded_ddp.py:211-653, fairscale/nn/pipe/pipeline.py:224-240),
so existing trace tooling keeps working.
"""

from __future__ import annotations

from contextlib import contextmanager
import os
import statistics
import subprocess
import threading
import time
from typing import Any, Dict, Iterator, List, Optional

import torch
from torch.autograd.profiler import record_function

_NVTX = torch.cuda.is_available()


@contextmanager
def trace_range(name: str) -> Iterator[None]:
    """``record_function`` + NVTX range (NVTX only when CUDA is present)."""
    if _NVTX:
        torch.cuda.nvtx.range_push(name)
    try:
        with record_function(name):
            yield
    finally:
        if _NVTX:
            torch.cuda.nvtx.range_pop()


class EventTimer:
    """Accumulates CUDA-event timings per name without synchronising in the timed code; ``summary()`` synchronises."""

    def __init__(self) -> None:
        self._pairs: Dict[str, List[Any]] = {}

    @contextmanager
    def time(self, name: str) -> Iterator[None]:
        if not torch.cuda.is_available():
            t0 = time.perf_counter()
            yield
            self._pairs.setdefault(name, []).append((time.perf_counter() - t0) * 1e3)
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        self._pairs.setdefault(name, []).append((a, b))

    def summary(self) -> Dict[str, Dict[str, float]]:
        out = {}
        for name, items in self._pairs.items():
            ms = []
            for it in items:
                if isinstance(it, tuple):
                    it[1].synchronize()
                    ms.append(it[0].elapsed_time(it[1]))
                else:
                    ms.append(it)
            out[name] = {"count": len(ms), "mean_ms": statistics.mean(ms), "std_ms": statistics.pstdev(ms) if len(ms) > 1 else 0.0,
                         "total_ms": sum(ms)}
        return out

    def reset(self) -> None:
        self._pairs.clear()


# ------------------------------------------------------------------------------------------------
# Step breakdown of the data-parallel wrappers: time of every collective on its own stream and the time the
# compute stream spent waiting for one ("exposed").  Off unless ``FSB200_COMM_TRACE=1`` or ``enable_comm_trace()``.
# ------------------------------------------------------------------------------------------------
_COMM_TRACE: Optional["EventTimer"] = None


def enable_comm_trace(on: bool = True) -> Optional["EventTimer"]:
    """Switch the collective / exposed-wait timers on (returns the shared :class:`EventTimer`) or off."""
    global _COMM_TRACE
    _COMM_TRACE = EventTimer() if on else None
    return _COMM_TRACE


def comm_trace() -> Optional["EventTimer"]:
    global _COMM_TRACE
    if _COMM_TRACE is None and os.environ.get("FSB200_COMM_TRACE", "0") == "1":
        _COMM_TRACE = EventTimer()
    return _COMM_TRACE


@contextmanager
def comm_range(name: str) -> Iterator[None]:
    """Time the enclosed launches on the current stream under ``name`` when the breakdown is enabled (no-op otherwise)."""
    t = comm_trace()
    if t is None:
        yield
        return
    with t.time(name):
        yield


class device_timer:
    """Times a block on the device (CUDA events on the current stream; host clock without a GPU) and, in a distributed
    job, reports the slowest rank: every multi-GPU number is a maximum over ranks, never one rank's wall clock.

        with device_timer(steps=4) as t:
            for _ in range(4): step()
        t.ms_per_step      # identical on every rank

    The block is bracketed by a barrier and a device synchronisation on both sides.
    """

    def __init__(self, steps: int = 1, group: Any = None) -> None:
        self.steps = steps
        self.group = group
        self.ms = 0.0
        self.ms_per_step = 0.0
        self._cuda = torch.cuda.is_available()

    def _fence(self) -> None:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            dist.barrier(group=self.group)
        if self._cuda:
            torch.cuda.synchronize()

    def __enter__(self) -> "device_timer":
        self._fence()
        if self._cuda:
            self._a, self._b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._a.record()
        else:
            self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc: Any) -> None:
        import torch.distributed as dist

        if self._cuda:
            self._b.record()
            self._b.synchronize()
            local = float(self._a.elapsed_time(self._b))
        else:
            local = (time.perf_counter() - self._t0) * 1e3
        if exc[0] is None and dist.is_available() and dist.is_initialized():
            t = torch.tensor([local], dtype=torch.float64, device="cuda" if (self._cuda and dist.get_backend(self.group) == "nccl") else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            local = float(t.item())
        self.ms = local
        self.ms_per_step = local / max(self.steps, 1)


@contextmanager
def chrome_trace(path: str, with_cuda: bool = True) -> Iterator[Any]:
    """Profile the block with ``torch.profiler`` and write a Chrome / Perfetto trace to ``path``."""
    acts = [torch.profiler.ProfilerActivity.CPU]
    if with_cuda and torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(activities=acts) as prof:
        yield prof
    prof.export_chrome_trace(path)


class ClockSampler:
    """Samples ``nvidia-smi`` SM clocks and throttle reasons of one GPU in a background thread (read-only queries)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0, period_s: float = 0.2) -> None:
        self.index, self.period = index, period_s
        self.samples: List[List[str]] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self) -> "ClockSampler":
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc: Any) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=6)

    def summary(self) -> Dict[str, Any]:
        sm = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(s) > 3 + i and s[3 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": float(self.samples[0][1]) if self.samples and self.samples[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(self.samples)}
