"""Tensor-parallel Llama-style LM benchmark (model_parallel layers, sequence-parallel fused all-gather->GEMM /
GEMM->reduce-scatter kernels): tokens/s of a training step with every GPU of the node in one model-parallel group.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/tp.py [--layers 32] [--unfused]

Device-timed with CUDA events, max over ranks.  ``--unfused`` routes the same model through NCCL collectives + the plain
GEMM (FSB200_COMM=nccl) for comparison.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--d_model", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--unfused", action="store_true")
    args = ap.parse_args()
    if args.unfused:
        os.environ["FSB200_COMM"] = "nccl"
    from fairscale_b200.models.tp_llama import TPLlama, TPLlamaConfig
    from fairscale_b200.nn.model_parallel import initialize_model_parallel
    from fairscale_b200.optim import FusedAdam
    from fairscale_b200.parallel import nvlink

    rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    initialize_model_parallel(world)
    from fairscale_b200.nn.model_parallel import get_model_parallel_group

    if world > 1 and not args.unfused:
        T = args.batch * args.seq
        heap_mb = (T * max(args.d_model, 3 * args.d_model // world, 2 * args.ffn // world) * 2 * 6 >> 20) + 256
        ws = nvlink.enable(get_model_parallel_group(), dev, staging_mb=64, heap_mb=heap_mb)
        from fairscale_b200.parallel import symm

        symm.register_workspace(get_model_parallel_group(), ws)
    torch.manual_seed(0)
    cfg = TPLlamaConfig(args.vocab, args.d_model, args.heads, args.layers, args.ffn, args.seq)
    model = TPLlama(cfg).to(dev).to(torch.bfloat16)
    opt = FusedAdam(model.parameters(), lr=1e-4)
    g = torch.Generator(device=dev).manual_seed(1)
    toks = torch.randint(0, args.vocab, (args.batch, args.seq + 1), device=dev, generator=g)
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()

    def step():
        loss = model(x, y)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    for _ in range(args.warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        loss = step()
    b.record()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if dist.get_rank() == 0:
        print(json.dumps({"benchmark": "tp_llama", "world": world, "fused": not args.unfused, "layers": args.layers, "ms_per_step": round(float(ms), 2),
                          "tokens_per_s": round(args.batch * args.seq / float(ms) * 1e3, 1), "loss": float(loss.detach()),
                          "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2)}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
