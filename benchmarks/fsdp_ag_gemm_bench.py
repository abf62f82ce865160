"""FSDP's parameter all-gather fused with the first GEMM that consumes the gathered weights, against the unfused routes.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29551 \\
        benchmarks/fsdp_ag_gemm_bench.py [--tokens 16384 --hidden 2048 --ffn 8192]

The flat parameter is that of one block of the flagship GPT (QKV weight first, 12 d^2 + small parameters in total); the
product is the QKV projection ``[tokens, d] x [3d, d]^T``.  Timed (CUDA events on the device with the host's enqueue hidden behind a spin kernel, max over ranks, L2 flushed
between iterations): the fused weight-gather GEMM with the copy-engine transport (per-piece arrival flags, the default) and with
copy CTAs inside the GEMM launch; copy-engine all-gather followed by the GEMM; NCCL all-gather followed by the
GEMM.  Roofline of the fused kernel: the slower of FLOPs / measured bf16 peak and the bytes that must enter this GPU over
NVLink / 770 GB/s (measured peer copy).
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
from fairscale_b200.utils.failure import check_device_status  # noqa: E402


def _peak():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path)).get("bf16_tflops", 1590.0)), "measured"
    except Exception:
        return 1590.0, "fallback"


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    total = 0.0
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
        total += a.elapsed_time(b)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() * 1e3  # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if "RANK" in os.environ:
        dist.init_process_group("nccl", device_id=dev)
    else:
        import socket

        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        dist.init_process_group("nccl", rank=0, world_size=1, init_method=f"tcp://127.0.0.1:{port}", device_id=dev)
    world, rank = dist.get_world_size(), dist.get_rank()
    d, f, T = args.hidden, args.ffn, args.tokens
    N, K = 3 * d, d
    total = 4 * d * d + 2 * d * f + 9 * d + f  # one block: qkv, proj, fc1, fc2 weights + biases + two LayerNorms
    n = -(-total // (world * 8)) * 8
    ws = nvlink.enable(None, dev, staging_mb=8, heap_mb=(2 * n >> 20) + 64)
    shard = ws.alloc_tensor((n,), torch.bfloat16).normal_(0, 0.02)
    full = torch.empty(n * world, device=dev, dtype=torch.bfloat16)
    x = (torch.randn(T, K, device=dev) * 0.5).bfloat16()
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device=dev)
    peak, src = _peak()
    flops = 2.0 * T * N * K
    nv_bytes = (world - 1) * n * 2.0
    ideal_us = max(flops / (peak * 1e12), nv_bytes / 770e9) * 1e6

    def fused():
        fused_tp.weight_gather_gemm(ws, x, shard, full, 0, N, K, None, engine="dma")

    def fused_sm():
        fused_tp.weight_gather_gemm(ws, x, shard, full, 0, N, K, None, engine="sm")

    def dma_then_gemm():
        ws.all_gather_engine = "dma"
        ws.all_gather(full, shard)
        gemm_ops.linear_forward(x, full[: N * K].view(N, K), None)

    def nccl_then_gemm():
        dist.all_gather_into_tensor(full, shard)
        gemm_ops.linear_forward(x, full[: N * K].view(N, K), None)

    def gemm_only():
        gemm_ops.linear_forward(x, full[: N * K].view(N, K), None)

    res = {"fused_us": timed(fused, args.iters, flush), "fused_sm_copy_us": timed(fused_sm, args.iters, flush), "dma_allgather_plus_gemm_us": timed(dma_then_gemm, args.iters, flush),
           "nccl_allgather_plus_gemm_us": timed(nccl_then_gemm, args.iters, flush), "gemm_alone_us": timed(gemm_only, args.iters, flush)}
    check_device_status(dev)
    if rank == 0:
        out = {"op": "fsdp_ag_gemm", "world": world, "M": T, "N": N, "K": K, "flat_param_mb": round(n * world * 2 / 2**20, 1),
               "nvlink_mb_per_gpu": round(nv_bytes / 2**20, 1), **{k: round(v, 1) for k, v in res.items()},
               "roofline_us": round(ideal_us, 1), "roofline_frac": round(ideal_us / res["fused_us"], 3), "peak_source": src,
               "speedup_vs_dma": round(res["dma_allgather_plus_gemm_us"] / res["fused_us"], 3),
               "speedup_vs_nccl": round(res["nccl_allgather_plus_gemm_us"] / res["fused_us"], 3)}
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
