"""MEVO (tiled projection + softmax + NLL) against the un-tiled baseline: time and peak memory over a few shapes
(reference driver: benchmarks/experimental/benchmark_mevo.py:21-174).

    python benchmarks/experimental/benchmark_mevo.py [--dry_run]
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from fairscale_b200.experimental.nn import BaselineSoftmaxNllLoss, MemoryEfficientVocabOutput  # noqa: E402
from fairscale_b200.experimental.nn.mevo import get_data  # noqa: E402

SHAPES = [((1024, 128), (128, 256008)), ((4096, 1024), (1024, 50304)), ((8192, 2048), (2048, 50304))]


def run(kernel_cls, shape, dtype, device, tile_factor):
    x, w, t = get_data(shape, dtype=dtype, device=device)
    mod = kernel_cls(w, tile_factor=tile_factor)
    if device == "cuda":
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(3):
        x.grad = w.grad = None
        loss = mod(x, t)
        loss.backward()
    if device == "cuda":
        torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / 3
    peak = torch.cuda.max_memory_allocated() if device == "cuda" else 0
    return dt, peak, float(loss.detach())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dry_run", action="store_true")
    ap.add_argument("--tile_factor", type=int, default=16)
    args = ap.parse_args()
    device = "cuda" if torch.cuda.is_available() else "cpu"
    dtype = torch.float16 if device == "cuda" else torch.float32
    shapes = [((64, 32), (32, 1000))] if args.dry_run else SHAPES
    for shape in shapes:
        tb, mb, lb = run(BaselineSoftmaxNllLoss, shape, dtype, device, 0)
        tm, mm, lm = run(MemoryEfficientVocabOutput, shape, dtype, device, args.tile_factor)
        print(json.dumps({"benchmark": "mevo", "shape": shape, "baseline_ms": round(tb * 1e3, 2), "mevo_ms": round(tm * 1e3, 2),
                          "baseline_peak_mb": mb >> 20, "mevo_peak_mb": mm >> 20, "loss_baseline": lb, "loss_mevo": lm}))


if __name__ == "__main__":
    main()
