"""Per-step metrics as JSON lines: throughput, bytes moved by each kind of collective, achieved fraction of a roofline.

The reference only logs through Python ``logging`` and prints words/s in its benchmark scripts (benchmarks/fsdp.py:221-241);
it has no metrics backend.  ``StepMetrics`` listens to the collective front-end (:mod:`fairscale_b200.parallel.comm`),
so every all-gather / reduce-scatter / all-reduce / all-to-all / broadcast / reduce issued by FSDP, ShardedDDP, OSS, the
tensor-parallel layers and the MoE layer is counted with its payload size, whichever transport carries it.
"""

from __future__ import annotations

import json
import time
from typing import IO, Any, Dict, Optional

import torch

from ..parallel import comm


def _nbytes(t: Any) -> int:
    return int(t.numel() * t.element_size()) if torch.is_tensor(t) else 0


class StepMetrics:
    """Collects one record per training step.

    Args:
        sink: a text stream (one JSON object per line is written to it) or ``None`` to only keep ``last``.
        tokens_per_step: used for ``tokens_per_s``; may also be passed to :meth:`end_step`.
        roofline_ms: time the step would take at the roofline chosen by the caller (e.g. FLOPs / measured GEMM peak, or
            NVLink bytes / link bandwidth, whichever is slower); gives ``roofline_fraction``.
        device_timing: time steps with CUDA events (synchronises in :meth:`end_step`) instead of the host clock.
    """

    def __init__(self, sink: Optional[IO[str]] = None, tokens_per_step: Optional[int] = None, roofline_ms: Optional[float] = None,
                 device_timing: Optional[bool] = None) -> None:
        self.sink = sink
        self.tokens_per_step = tokens_per_step
        self.roofline_ms = roofline_ms
        self.device_timing = torch.cuda.is_available() if device_timing is None else device_timing
        self.last: Dict[str, Any] = {}
        self._step = 0
        self._bytes: Dict[str, int] = {}
        self._calls: Dict[str, int] = {}
        self._t0 = 0.0
        self._ev: Any = None
        self._listening = False

    # ------------------------------------------------------------------ listener
    def _on_collective(self, kind: str, group: Any, out: Any, inp: Any) -> None:
        # payload = the larger side: the gathered output of an all-gather, the full input of a reduce-scatter
        self._bytes[kind] = self._bytes.get(kind, 0) + max(_nbytes(out), _nbytes(inp))
        self._calls[kind] = self._calls.get(kind, 0) + 1

    def start(self) -> "StepMetrics":
        if not self._listening:
            comm.add_listener(self._on_collective)
            self._listening = True
        return self

    def stop(self) -> None:
        if self._listening:
            comm.remove_listener(self._on_collective)
            self._listening = False

    def __enter__(self) -> "StepMetrics":
        return self.start()

    def __exit__(self, *exc: Any) -> None:
        self.stop()

    # ------------------------------------------------------------------ steps
    def begin_step(self) -> None:
        self._bytes, self._calls = {}, {}
        if self.device_timing:
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()
        else:
            self._t0 = time.perf_counter()

    def end_step(self, tokens: Optional[int] = None, **extra: Any) -> Dict[str, Any]:
        if self.device_timing:
            self._ev[1].record()
            self._ev[1].synchronize()
            ms = float(self._ev[0].elapsed_time(self._ev[1]))
        else:
            ms = (time.perf_counter() - self._t0) * 1e3
        tokens = tokens if tokens is not None else self.tokens_per_step
        rec: Dict[str, Any] = {"step": self._step, "ms": round(ms, 3), "comm_bytes": dict(self._bytes), "comm_calls": dict(self._calls)}
        if tokens is not None and ms > 0:
            rec["tokens_per_s"] = round(tokens / ms * 1e3, 1)
        if self.roofline_ms is not None and ms > 0:
            rec["roofline_fraction"] = round(self.roofline_ms / ms, 4)
        if torch.cuda.is_available():
            rec["peak_mem_bytes"] = int(torch.cuda.max_memory_allocated())
        rec.update(extra)
        self.last = rec
        self._step += 1
        if self.sink is not None:
            self.sink.write(json.dumps(rec) + "\n")
            self.sink.flush()
        return rec
