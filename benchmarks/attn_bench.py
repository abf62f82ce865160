"""Run the tcgen05 causal attention (forward + backward) a few times on one shape and print CUDA-event timings next to
cuDNN / flash SDPA through PyTorch (small driver for `ncu` captures and quick comparisons).

    python benchmarks/attn_bench.py --b 8 --s 2048 --h 16 --d 128 --iters 5
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

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


def timed_loop(call, iters):
    """Mean device time of `iters` back-to-back calls issued behind a spin kernel, so that host launch latency (Python,
    tensor-map encoding, allocation) stays out of the measurement."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(2):
        call()
    torch.cuda.synchronize()
    torch.cuda._sleep(4_000_000)
    a.record()
    for _ in range(iters):
        call()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def ours(iters):
    """The native kernels called directly (what the autograd function of ops/attention_native.py launches)."""
    from fairscale_b200.ops import _bind, attention_native

    attention_native._bind_sigs()
    q = qkv.detach()
    o = torch.empty(a.b, a.s, a.h * a.d, dtype=q.dtype, device=dev)
    lse = torch.empty(a.b, a.h, a.s, dtype=torch.float32, device=dev)
    delta = torch.empty(2, a.b, a.h, a.s, dtype=torch.float32, device=dev)
    dqkv = torch.empty_like(q)
    scale = a.d ** -0.5
    st, stream = _bind.status_ptr(dev), _bind.stream_ptr(dev)
    f = timed_loop(lambda: _bind.call("fsb_attn_fwd", q.data_ptr(), o.data_ptr(), lse.data_ptr(), a.b, a.s, a.h, a.d, scale, st, stream), iters)
    g = timed_loop(lambda: _bind.call("fsb_attn_bwd", q.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                                      dqkv.data_ptr(), a.b, a.s, a.h, a.d, scale, st, stream, launches=3), iters)
    return f, g


def sdpa(iters):
    """cuDNN / flash attention through scaled_dot_product_attention, with the permute it needs on packed QKV."""
    def fwd():
        q, k, v = qkv.view(a.b, a.s, 3, a.h, a.d).permute(2, 0, 3, 1, 4)
        return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(a.b, a.s, a.h * a.d)

    with torch.no_grad():
        f = timed_loop(fwd, iters)
    o = fwd()
    g = timed_loop(lambda: torch.autograd.grad(o, qkv, do, retain_graph=True), iters)
    return f, g


flops_f = 4.0 * a.b * a.h * a.s * a.s * a.d / 2
f, b = ours(a.iters)
print(f"ours  B={a.b} S={a.s} H={a.h} D={a.d}: fwd {f * 1e3:.1f} us ({flops_f / f / 1e9:.0f} TFLOP/s)  bwd {b * 1e3:.1f} us ({2.5 * flops_f / b / 1e9:.0f} TFLOP/s)")
if not a.no_sdpa:
    f, b = sdpa(a.iters)
    print(f"sdpa  (incl. its permute / cat glue): fwd {f * 1e3:.1f} us ({flops_f / f / 1e9:.0f} TFLOP/s)  bwd {b * 1e3:.1f} us ({2.5 * flops_f / b / 1e9:.0f} TFLOP/s)")
