"""Run the tcgen05 causal attention (forward + backward) a few times on one shape and print CUDA-event timings next to
cuDNN / flash SDPA through PyTorch (small driver for `ncu` captures and quick comparisons).

    python benchmarks/attn_one.py --b 8 --s 2048 --h 16 --d 128 --iters 5
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fairscale_b200.ops.attention import causal_attention  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--b", type=int, default=8)
ap.add_argument("--s", type=int, default=2048)
ap.add_argument("--h", type=int, default=16)
ap.add_argument("--d", type=int, default=128)
ap.add_argument("--iters", type=int, default=5)
ap.add_argument("--no-sdpa", action="store_true")
a = ap.parse_args()
dev = torch.device("cuda", 0)
qkv = (torch.randn(a.b, a.s, 3 * a.h * a.d, device=dev) * 0.5).bfloat16().requires_grad_()
do = torch.randn(a.b, a.s, a.h * a.d, device=dev).bfloat16()


def run(fn, iters):
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    f = b = 0.0
    for i in range(iters):
        qkv.grad = None
        ev[0].record()
        o = fn()
        ev[1].record()
        o.backward(do)
        ev[2].record()
        torch.cuda.synchronize()
        if i >= iters // 2:
            f += ev[0].elapsed_time(ev[1])
            b += ev[1].elapsed_time(ev[2])
    n = iters - iters // 2
    return f / n, b / n


def sdpa():
    q, k, v = qkv.view(a.b, a.s, 3, a.h, a.d).permute(2, 0, 3, 1, 4)
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(a.b, a.s, a.h * a.d)


flops_f = 4.0 * a.b * a.h * a.s * a.s * a.d / 2
f, b = run(lambda: causal_attention(qkv, a.h), a.iters)
print(f"ours  B={a.b} S={a.s} H={a.h} D={a.d}: fwd {f * 1e3:.1f} us ({flops_f / f / 1e9:.0f} TFLOP/s)  bwd {b * 1e3:.1f} us ({2.5 * flops_f / b / 1e9:.0f} TFLOP/s)")
if not a.no_sdpa:
    f, b = run(sdpa, a.iters)
    print(f"sdpa  (incl. its permute / cat glue): fwd {f * 1e3:.1f} us ({flops_f / f / 1e9:.0f} TFLOP/s)  bwd {b * 1e3:.1f} us ({2.5 * flops_f / b / 1e9:.0f} TFLOP/s)")
