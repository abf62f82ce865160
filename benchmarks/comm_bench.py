"""Bandwidth of the in-kernel NVLink collectives against NCCL on the same buffers.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29541 \
        benchmarks/comm_bench.py [--mb 16 64 256]

For every size it times all-gather and reduce-scatter (CUDA events, max over ranks, inputs resident in the symmetric
heap) and prints the per-GPU receive bandwidth: bytes that have to cross NVLink into one GPU divided by the time,
which is the figure to hold against the measured 770 GB/s per direction of a peer copy on this hardware.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fairscale_b200.parallel import nvlink  # noqa: E402
from fairscale_b200.utils.failure import check_device_status  # noqa: E402


def timed(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def one_rank(args):
    import socket

    from fairscale_b200.optim import FusedAdam

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    dist.init_process_group("nccl", rank=0, world_size=1, init_method=f"tcp://127.0.0.1:{port}", device_id=dev)
    mb = max(args.mb)
    n = (mb << 20) // 2 // 64 * 64  # bf16 elements
    ws = nvlink.enable(None, dev, staging_mb=8, heap_mb=8 * mb + 64)
    ws.enable_grad_windows(2 * n + 1024, 2)
    shard = ws.alloc_tensor((n,), torch.bfloat16).normal_()
    out_full = torch.empty(n, dtype=torch.bfloat16, device=dev)
    out_shard = torch.empty(n, dtype=torch.float32, device=dev)
    p = torch.nn.Parameter(torch.randn(n, device=dev))
    opt = FusedAdam([p], lr=1e-3)
    copy = ws.alloc_tensor((n,), torch.bfloat16)
    opt.param_copies[p] = copy
    rows, M = n // 1024, 1024
    x = torch.randn(rows, M, device=dev).bfloat16()
    land = ws.alloc_tensor((rows, M), torch.bfloat16)
    dst_rank = torch.zeros(rows, dtype=torch.int32, device=dev)
    dst_row = torch.randperm(rows, device=dev).to(torch.int32)
    w = torch.rand(rows, device=dev)
    back = torch.empty_like(x)

    def step():
        g = ws.grad_window(n, torch.bfloat16, dev)
        g.normal_()
        ws.all_gather_engine = "kernel"
        ws.all_gather(out_full, shard)
        ws.reduce_scatter(out_shard, g, scale=1.0)
        g2 = ws.grad_window(n, torch.bfloat16, dev)
        g2.normal_()
        opt.reduce_scatter_step(p, ws, g2, 1.0)
        ws.moe_scatter_rows(land, x, dst_rank, dst_row, None, 1)
        ws.moe_gather_rows(land, back, dst_rank, dst_row, w, 1)

    ms = timed(step, args.iters)
    check_device_status(dev)
    print(f"one rank, {mb} MB per collective: {ms * 1e3:.1f} us per iteration of all-gather + reduce-scatter + reduce-scatter-Adam + "
          f"MoE scatter + MoE gather", flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, nargs="+", default=[16, 100, 256], help="size of the full (gathered / unreduced) tensor in MB")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--one-rank", action="store_true",
                    help="a group of one rank in this process (plain `python`, no launcher): every collective kernel, the fused "
                         "reduce-scatter + Adam and the MoE row scatter / gather run once per iteration on local memory - the case "
                         "to capture with a profiler, which must never wrap a multi-rank launch")
    args = ap.parse_args()
    if args.one_rank:
        return one_rank(args)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ws = nvlink.enable(None, dev, staging_mb=8, heap_mb=2 * max(args.mb) + 64)
    for mb in args.mb:
        n = (mb << 20) // 2 // world // 64 * 64  # bf16 elements per rank
        shard = ws.alloc_tensor((n,), torch.bfloat16).normal_()
        full_in = ws.alloc_tensor((n * world,), torch.bfloat16).normal_()
        out_full = torch.empty(n * world, dtype=torch.bfloat16, device=dev)
        out_shard = torch.empty(n, dtype=torch.float32, device=dev)
        out_shard_bf = torch.empty(n, dtype=torch.bfloat16, device=dev)
        cross = 2.0 * n * (world - 1)  # bytes entering one GPU over NVLink, both collectives
        def ag(engine):
            ws.all_gather_engine = engine
            return timed(lambda: ws.all_gather(out_full, shard), args.iters)

        res = {
            "ag_nvlink": ag("kernel"),
            "ag_dma": ag("dma"),
            "ag_nccl": timed(lambda: dist.all_gather_into_tensor(out_full, shard), args.iters),
            "rs_nvlink": timed(lambda: ws.reduce_scatter(out_shard, full_in, scale=1.0 / world), args.iters),
            "rs_nccl": timed(lambda: dist.reduce_scatter_tensor(out_shard_bf, full_in), args.iters),
        }
        if rank == 0:
            print(f"{mb:4d} MB over {world} GPUs: " + "  ".join(f"{k} {v * 1e3:7.1f} us ({cross / v / 1e6:6.1f} GB/s)" for k, v in res.items()), flush=True)
    check_device_status(dev)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
