"""Time the tcgen05 GEMM against torch.matmul (cuBLAS) on the linear-layer shapes of the flagship models.

    python benchmarks/gemm_bench.py [--json out.json]
    python benchmarks/gemm_bench.py --shape 8192 8192 2048 --mode fwd --iters 4     # one product, a few launches (profiler captures)

Each product is timed with CUDA events over `iters` back-to-back launches after warm-up; operands are
rotated through enough distinct buffers to exceed the 126 MB L2.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fairscale_b200.ops.gemm import linear_dgrad, linear_forward, linear_wgrad  # noqa: E402

SHAPES = [  # (tokens M, out N, in K)
    (16384, 6144, 2048), (16384, 2048, 2048), (16384, 8192, 2048), (16384, 2048, 8192), (16384, 50304, 2048),
    (8192, 4096, 1024), (8192, 1024, 4096), (32768, 1536, 4096), (32768, 4096, 512),
]


def timeit(fn, sets, iters=20, warmup=5):
    for i in range(warmup):
        fn(*sets[i % len(sets)])
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(iters):
        fn(*sets[i % len(sets)])
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters


def run_one(m: int, n: int, k: int, mode: str, iters: int) -> None:
    """A few launches of one product (with its fused epilogue variants); prints the time of the last launch."""
    dev = torch.device("cuda", 0)
    x = torch.randn(m, k, device=dev).bfloat16()
    w = torch.randn(n, k, device=dev).bfloat16()
    dy = torch.randn(m, n, device=dev).bfloat16()
    bias = torch.randn(n, device=dev).bfloat16()
    pre = torch.randn(m, k, device=dev).bfloat16()
    calls = {
        "fwd": lambda: linear_forward(x, w),
        "fwd_gelu": lambda: linear_forward(x, w, bias, gelu=True, save_pre_activation=True),
        "dgrad": lambda: linear_dgrad(dy, w),
        "dgrad_dgelu": lambda: linear_dgrad(dy, w, dgelu_pre=pre),
        "wgrad": lambda: linear_wgrad(dy, x),
    }
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(iters):
        if i == iters - 1:
            t0.record()
        calls[mode]()
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    print(f"{mode} M={m} N={n} K={k}: {ms * 1e3:.1f} us, {2.0 * m * n * k / ms / 1e9:.0f} TFLOP/s")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), default=None, help="run only this product")
    ap.add_argument("--mode", default="fwd", choices=["fwd", "fwd_gelu", "dgrad", "dgrad_dgelu", "wgrad"])
    args = ap.parse_args()
    if args.shape is not None:
        run_one(*args.shape, args.mode, args.iters)
        return
    dev = torch.device("cuda", 0)
    rows = []
    for M, N, K in SHAPES:
        bytes_per_set = 2 * (M * K + N * K + M * N)
        nsets = max(2, min(8, (300 << 20) // bytes_per_set + 1))
        xs = [torch.randn(M, K, device=dev).bfloat16() for _ in range(nsets)]
        ws = [torch.randn(N, K, device=dev).bfloat16() for _ in range(nsets)]
        dys = [torch.randn(M, N, device=dev).bfloat16() for _ in range(nsets)]
        flops = 2.0 * M * N * K
        res = {"M": M, "N": N, "K": K}
        for name, mine, lib, sets in [
            ("fwd", lambda x, w, dy: linear_forward(x, w), lambda x, w, dy: x @ w.t(), list(zip(xs, ws, dys))),
            ("dgrad", lambda x, w, dy: linear_dgrad(dy, w), lambda x, w, dy: dy @ w, list(zip(xs, ws, dys))),
            ("wgrad", lambda x, w, dy: linear_wgrad(dy, x), lambda x, w, dy: dy.t() @ x, list(zip(xs, ws, dys))),
        ]:
            t_mine = timeit(mine, sets, args.iters)
            t_lib = timeit(lib, sets, args.iters)
            res[name] = {"ours_ms": round(t_mine, 4), "cublas_ms": round(t_lib, 4), "ours_tflops": round(flops / t_mine / 1e9, 1),
                         "cublas_tflops": round(flops / t_lib / 1e9, 1)}
        print(json.dumps(res), flush=True)
        rows.append(res)
        del xs, ws, dys
        torch.cuda.empty_cache()
    if args.json:
        json.dump(rows, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
