"""Time the fused tensor-parallel kernels against the unfused baseline (NCCL collective + the same tcgen05 GEMM).

Launch: ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/fused_tp_bench.py``
(or ``python benchmarks/fused_tp_bench.py --tokens 8192 --hidden 2048 --ffn 4096 --iters 2`` for a one-rank run on GPU 0).
CUDA-event timing after warm-up, max over ranks; a buffer larger than L2 is rewritten between iterations.
Roofline per op: the slower of FLOPs / measured bf16 GEMM peak and NVLink bytes / 770 GB/s (measured peer copy).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fairscale_b200.ops import gemm as gemm_ops  # noqa: E402
from fairscale_b200.parallel import fused_tp, nvlink  # noqa: E402


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        return float(d.get("bf16_tflops", 1590.0)), "measured"
    except Exception:
        return 1590.0, "fallback"


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        flush.add_(1)
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(3_000_000)  # ~1.5 ms of device time: the host enqueues fn() behind it, so a..b is device time only
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    t = torch.tensor([sorted(times)[len(times) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t) * 1e3  # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=12288)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(rank)
    if "RANK" in os.environ:
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    else:
        # started plainly (no launcher): a one-rank group on GPU 0.  The kernels then show their structure (copy CTAs and
        # tcgen05 CTAs in one launch) without any peer, which is what a single-GPU profiler capture needs.
        import socket

        with socket.socket() as sock:
            sock.bind(("127.0.0.1", 0))
            port = sock.getsockname()[1]
        dist.init_process_group("nccl", rank=0, world_size=1, init_method=f"tcp://127.0.0.1:{port}", device_id=torch.device("cuda", 0))
    world = dist.get_world_size()
    dev = torch.device("cuda", rank)
    T, H, F = args.tokens, args.hidden, args.ffn // world
    ws = nvlink.enable(None, dev, staging_mb=16, heap_mb=(T * max(H, F) * 2 * 2 >> 20) + 64)
    peak, src = _peaks()
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device=dev)
    xs = (torch.randn(T // world, H, device=dev) * 0.1).bfloat16()
    w1 = (torch.randn(F, H, device=dev) * 0.02).bfloat16()
    full = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    xa = (torch.randn(T, F, device=dev) * 0.1).bfloat16()
    w2 = (torch.randn(H, F, device=dev) * 0.02).bfloat16()
    shard = torch.empty(T // world, H, device=dev, dtype=torch.bfloat16)

    def ag_unfused():
        dist.all_gather_into_tensor(full, xs)
        gemm_ops.linear_forward(full, w1, None)

    def rs_unfused():
        y, _ = gemm_ops.linear_forward(xa, w2, None)
        dist.reduce_scatter_tensor(shard, y)

    rows = []
    flops = 2.0 * T * H * F
    nv_bytes = (world - 1) / world * T * H * 2
    ideal_us = max(flops / (peak * 1e12), nv_bytes / 770e9) * 1e6
    for name, fused, unfused in (("ag_gemm", lambda: fused_tp.ag_gemm(ws, xs, w1, None, engine="dma"), ag_unfused),
                                 ("ag_gemm_sm_copy", lambda: fused_tp.ag_gemm(ws, xs, w1, None, engine="sm"), ag_unfused),
                                 ("gemm_rs", lambda: fused_tp.gemm_rs(ws, xa, w2, None), rs_unfused)):
        tf, tu = _time(fused, args.iters, flush), _time(unfused, args.iters, flush)
        rows.append({"op": name, "world": world, "M": T, "N": F if name.startswith("ag_gemm") else H, "K": H if name.startswith("ag_gemm") else F,
                     "fused_us": round(tf, 1), "unfused_us": round(tu, 1), "speedup": round(tu / tf, 3),
                     "fused_tflops": round(flops / tf / 1e6, 1), "roofline_us": round(ideal_us, 1),
                     "roofline_frac": round(ideal_us / tf, 3), "peak_source": src, "comm_ctas": os.environ.get("FSB200_FUSED_COMM_CTAS", "auto")})
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
