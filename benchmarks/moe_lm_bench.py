"""Expert-parallel MoE language-model benchmark: top-2 gating, `--experts-per-gpu` experts on every rank, dense parts
data parallel.  Default shape: 12 layers (every other feed-forward is an MoE layer), d_model 1024, FFN 4096, 16 heads,
sequence 1024, batch 8 per GPU, bf16.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/moe_lm_bench.py
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/moe_lm_bench.py --impl reference

`--impl ours` runs `fairscale_b200.models.moe_lm.MoELM` (index routing kernels, NVLink row scatter / gather for
dispatch and combine, one grouped tcgen05 launch per expert layer, fused Adam).  `--impl reference` builds the same
architecture from torch.nn modules around the UNMODIFIED reference `MOELayer` / `Top2Gate` (dense one-hot einsum
dispatch, NCCL all_to_all, a Python loop over the local experts) under bf16 autocast, as the reference's own
benchmarks/moe.py:28-122 does, with torch's fused Adam.  Both arms synchronise the dense gradients with torch DDP
(expert parameters excluded).  Synthetic tokens, random-init weights; device-timed with CUDA events, max over ranks.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
from torch import nn
from torch.nn import functional as F
from torch.nn.parallel import DistributedDataParallel as DDP

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


class _RefExpert(nn.Module):
    def __init__(self, d, ffn):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(d, ffn), nn.Linear(ffn, d)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x)))


class _RefBlock(nn.Module):
    def __init__(self, d, heads, ffn, moe):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.moe = moe
        if moe is None:
            self.ffn = _RefExpert(d, ffn)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, s, d))
        h = self.ln2(x)
        return x + (self.ffn(h) if self.moe is None else self.moe(h))


class _RefMoELM(nn.Module):
    def __init__(self, args, world):
        super().__init__()
        sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
        from fairscale.nn import MOELayer, Top2Gate  # the reference library, stock code path

        d = args.d_model
        self.wte, self.wpe = nn.Embedding(args.vocab, d), nn.Embedding(args.seq, d)
        blocks = []
        for i in range(args.layers):
            moe = None
            if i % 2 == 1:
                experts = nn.ModuleList([_RefExpert(d, args.ffn) for _ in range(args.experts_per_gpu)])
                moe = MOELayer(Top2Gate(d, args.experts_per_gpu * world), experts)
            blocks.append(_RefBlock(d, args.heads, args.ffn, moe))
        self.blocks = nn.ModuleList(blocks)
        self.ln_f, self.out = nn.LayerNorm(d), nn.Linear(d, args.vocab, bias=False)

    def forward(self, tokens, targets):
        x = self.wte(tokens) + self.wpe(torch.arange(tokens.shape[1], device=tokens.device))
        aux = 0.0
        for blk in self.blocks:
            x = blk(x)
            if blk.moe is not None:
                aux = aux + blk.moe.l_aux
        logits = self.out(self.ln_f(x))
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1)) + 0.01 * aux


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--d_model", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--ffn", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=8, help="sequences per GPU")
    ap.add_argument("--experts-per-gpu", type=int, default=8)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()

    rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    if "RANK" not in os.environ:
        os.environ.update(RANK="0", WORLD_SIZE="1", MASTER_ADDR="127.0.0.1", MASTER_PORT="29541")
    dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    torch.manual_seed(0)

    if args.impl == "ours":
        from fairscale_b200.models.moe_lm import MoELM, MoELMConfig
        from fairscale_b200.optim import FusedAdam
        from fairscale_b200.parallel import nvlink

        if world > 1:
            # three landing buffers of 2 * tokens rows per MoE layer (each layer keeps its own), plus room for the shared ones
            per_buffer = 2 * args.batch * args.seq * args.d_model * 2
            nvlink.enable(dist.group.WORLD, dev, staging_mb=64, heap_mb=((3 * args.layers + 4) * per_buffer >> 20) + 64)
        cfg = MoELMConfig(vocab_size=args.vocab, d_model=args.d_model, n_heads=args.heads, n_layers=args.layers, ffn=args.ffn,
                          max_seq=args.seq, num_local_experts=args.experts_per_gpu)
        model = MoELM(cfg).to(dev).to(torch.bfloat16)
        opt = FusedAdam(model.parameters(), lr=1e-4)
        ctx = torch.autocast("cuda", enabled=False)
    else:
        model = _RefMoELM(args, world).to(dev)
        opt = torch.optim.Adam(model.parameters(), lr=1e-4, fused=True)
        ctx = torch.autocast("cuda", dtype=torch.bfloat16)
    expert_names = [n for n, p in model.named_parameters() if getattr(p, "expert", False)]
    DDP._set_params_and_buffers_to_ignore_for_model(model, expert_names)
    ddp = DDP(model, device_ids=[rank]) if world > 1 else model

    g = torch.Generator(device=dev).manual_seed(1 + dist.get_rank())
    toks = torch.randint(0, args.vocab, (args.batch, args.seq + 1), device=dev, generator=g)
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()

    def step():
        with ctx:
            loss = ddp(x, y)
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
        print(json.dumps({"benchmark": "moe_lm", "impl": args.impl, "world": world, "experts": args.experts_per_gpu * world,
                          "layers": args.layers, "ms_per_step": round(float(ms), 2),
                          "tokens_per_s": round(world * args.batch * args.seq / float(ms) * 1e3, 1), "loss": float(loss.detach()),
                          "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2)}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
