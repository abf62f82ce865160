"""Run the fused all-gather->GEMM and GEMM->reduce-scatter kernels in a one-rank group (small driver for single-GPU
`ncu` captures of the kernels' structure: copy CTAs + tcgen05 CTAs in one launch).  Multi-GPU timing: fused_tp_bench.py.

    python benchmarks/fused_tp_one.py --tokens 8192 --hidden 2048 --ffn 4096 --iters 4
"""
import argparse
import os
import socket
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fairscale_b200 import _native  # noqa: E402
from fairscale_b200.parallel import fused_tp, nvlink  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--tokens", type=int, default=8192)
ap.add_argument("--hidden", type=int, default=2048)
ap.add_argument("--ffn", type=int, default=4096)
ap.add_argument("--iters", type=int, default=4)
a = ap.parse_args()
torch.cuda.set_device(0)
dev = torch.device("cuda", 0)
with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
dist.init_process_group("nccl", rank=0, world_size=1, init_method=f"tcp://127.0.0.1:{port}", device_id=dev)
ws = nvlink.enable(None, dev, staging_mb=16, heap_mb=(a.tokens * max(a.hidden, a.ffn) * 2 * 2 >> 20) + 64)
x = (torch.randn(a.tokens, a.hidden, device=dev) * 0.1).bfloat16()
w1 = (torch.randn(a.ffn, a.hidden, device=dev) * 0.02).bfloat16()
h = (torch.randn(a.tokens, a.ffn, device=dev) * 0.1).bfloat16()
w2 = (torch.randn(a.hidden, a.ffn, device=dev) * 0.02).bfloat16()
for name, fn, ref in (("ag_gemm", lambda: fused_tp.ag_gemm(ws, x, w1, None)[0], lambda: x.float() @ w1.float().t()),
                      ("gemm_rs", lambda: fused_tp.gemm_rs(ws, h, w2, None), lambda: h.float() @ w2.float().t())):
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(a.iters):
        if i == a.iters - 1:
            t0.record()
        y = fn()
    t1.record()
    torch.cuda.synchronize()
    err = float((y.float() - ref()).norm() / ref().norm())
    flops = 2.0 * a.tokens * a.hidden * a.ffn
    print(f"{name}: {t0.elapsed_time(t1) * 1e3:.1f} us, {flops / t0.elapsed_time(t1) / 1e9:.0f} TFLOP/s, rel err {err:.2e}, status {_native.read_status(dev)}")
dist.destroy_process_group()
