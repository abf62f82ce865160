"""Run one tcgen05 GEMM shape a few times (small driver for `ncu` captures of the GEMM kernels).

    python benchmarks/gemm_one.py --m 8192 --n 8192 --k 2048 --mode fwd --iters 4
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fairscale_b200.ops.gemm import linear_dgrad, linear_forward, linear_wgrad  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--m", type=int, default=8192)
ap.add_argument("--n", type=int, default=8192)
ap.add_argument("--k", type=int, default=2048)
ap.add_argument("--mode", default="fwd", choices=["fwd", "fwd_gelu", "dgrad", "dgrad_dgelu", "wgrad"])
ap.add_argument("--iters", type=int, default=4)
a = ap.parse_args()
dev = torch.device("cuda", 0)
x = torch.randn(a.m, a.k, device=dev).bfloat16()
w = torch.randn(a.n, a.k, device=dev).bfloat16()
dy = torch.randn(a.m, a.n, device=dev).bfloat16()
bias = torch.randn(a.n, device=dev).bfloat16()
pre = torch.randn(a.m, a.k, device=dev).bfloat16()
t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
for i in range(a.iters):
    if i == a.iters - 1:
        t0.record()
    if a.mode == "fwd":
        linear_forward(x, w)
    elif a.mode == "fwd_gelu":
        linear_forward(x, w, bias, gelu=True, save_pre_activation=True)
    elif a.mode == "dgrad_dgelu":
        linear_dgrad(dy, w, dgelu_pre=pre)
    elif a.mode == "dgrad":
        linear_dgrad(dy, w)
    else:
        linear_wgrad(dy, x)
t1.record()
torch.cuda.synchronize()
ms = t0.elapsed_time(t1)
print(f"{a.mode} M={a.m} N={a.n} K={a.k}: {ms:.4f} ms, {2.0 * a.m * a.n * a.k / ms / 1e9:.1f} TFLOP/s")
