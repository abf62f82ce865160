"""Tensor-parallel Llama-style LM benchmark (model_parallel layers, sequence-parallel fused all-gather->GEMM /
GEMM->reduce-scatter kernels): tokens/s of a training step with every GPU of the node in one model-parallel group.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/tp.py [--layers 32] [--unfused]

Device-timed with CUDA events, max over ranks.  ``--unfused`` routes the same model through NCCL collectives + the plain
GEMM (FSB200_COMM=nccl) for comparison.  ``--impl reference`` builds the same architecture from torch.nn modules around
the UNMODIFIED reference library's VocabParallelEmbedding / ColumnParallelLinear / RowParallelLinear /
vocab_parallel_cross_entropy (all-reduce based, cuBLAS, torch SDPA, torch fused Adam).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _rope_torch(qkv, theta):
    B, S, _, H, Dh = qkv.shape
    pos = torch.arange(S, device=qkv.device, dtype=torch.float32)
    inv = theta ** (-torch.arange(0, Dh, 2, device=qkv.device, dtype=torch.float32) / Dh)
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, :, None, None, :], ang.sin()[None, :, None, None, :]
    qk = qkv[:, :, :2].float()
    x1, x2 = qk[..., 0::2], qk[..., 1::2]
    rot = torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).flatten(-2)
    return torch.cat([rot.to(qkv.dtype), qkv[:, :, 2:]], dim=2)


def build_reference_tp_llama(args, world, dev):
    """The reference arm: nothing from fairscale_b200 on this path."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref"))
    from fairscale.nn.model_parallel import initialize_model_parallel as ref_init
    from fairscale.nn.model_parallel.cross_entropy import vocab_parallel_cross_entropy as ref_ce
    from fairscale.nn.model_parallel.layers import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding
    from torch import nn
    from torch.nn import functional as F

    ref_init(world)
    keep = lambda w: w  # noqa: E731  (weights are drawn on the GPU after construction: a CPU draw of 7 B values per rank takes minutes)
    d, heads = args.d_model, args.heads

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1, self.norm2 = nn.RMSNorm(d, eps=1e-6), nn.RMSNorm(d, eps=1e-6)
            self.qkv = ColumnParallelLinear(d, 3 * d, bias=False, gather_output=False, init_method=keep)
            self.proj = RowParallelLinear(d, d, bias=False, input_is_parallel=True, init_method=keep)
            self.gate_up = ColumnParallelLinear(d, 2 * args.ffn, bias=False, gather_output=False, init_method=keep)
            self.down = RowParallelLinear(args.ffn, d, bias=False, input_is_parallel=True, init_method=keep)

        def forward(self, x):
            B, S, _ = x.shape
            qkv = _rope_torch(self.qkv(self.norm1(x)).view(B, S, 3, heads // world, d // heads), 10000.0)
            q, k, v = qkv.permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + self.proj(a.transpose(1, 2).reshape(B, S, -1))
            g, u = self.gate_up(self.norm2(x)).chunk(2, dim=-1)
            return x + self.down(F.silu(g) * u)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = VocabParallelEmbedding(args.vocab, d, init_method=keep)
            self.blocks = nn.ModuleList([Block() for _ in range(args.layers)])
            self.norm = nn.RMSNorm(d, eps=1e-6)
            self.head = ColumnParallelLinear(d, args.vocab, bias=False, gather_output=False, init_method=keep)

        def forward(self, tokens, targets):
            x = self.embed(tokens)
            for blk in self.blocks:
                x = blk(x)
            logits = self.head(self.norm(x))
            return ref_ce(logits.float(), targets).mean()

    model = Model().to(dev).to(torch.bfloat16)
    torch.manual_seed(1234 + dist.get_rank())
    with torch.no_grad():
        for prm in model.parameters():
            if prm.dim() > 1:
                prm.normal_(0.0, 0.02)
            else:
                prm.fill_(1.0)
    return model


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
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
    rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    torch.manual_seed(0)
    if args.impl == "reference":
        model = build_reference_tp_llama(args, world, dev)
        opt = torch.optim.Adam(model.parameters(), lr=1e-4, fused=True)
    else:
        from fairscale_b200.models.tp_llama import TPLlama, TPLlamaConfig
        from fairscale_b200.nn.model_parallel import get_model_parallel_group, initialize_model_parallel
        from fairscale_b200.optim import FusedAdam
        from fairscale_b200.parallel import nvlink, symm

        initialize_model_parallel(world)
        if world > 1 and not args.unfused:
            T = args.batch * args.seq
            heap_mb = (T * max(args.d_model, 3 * args.d_model // world, 2 * args.ffn // world) * 2 * 6 >> 20) + 256
            ws = nvlink.enable(get_model_parallel_group(), dev, staging_mb=max(64, (T * args.d_model * 2 >> 20) + 16), heap_mb=heap_mb)
            symm.register_workspace(get_model_parallel_group(), ws)
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
        print(json.dumps({"benchmark": "tp_llama", "impl": args.impl, "world": world, "fused": not args.unfused, "layers": args.layers, "ms_per_step": round(float(ms), 2),
                          "tokens_per_s": round(args.batch * args.seq / float(ms) * 1e3, 1), "loss": float(loss.detach()),
                          "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2)}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
