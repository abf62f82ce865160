"""GPipe language-model benchmark over pipeline stages: 48 layers d2048 in 8 stages of 6, sequence 1024, global batch
256 in 32 micro-batches, bf16 (defaults; every size is a flag).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/pipe_lm_bench.py
    python benchmarks/pipe_lm_bench.py --impl reference --stages 8

`--impl ours`: one process per stage, `fairscale_b200.nn.pipe.AsyncPipe` over NCCL p2p (gloo with `--cpu`), the flagship
GPT blocks (tcgen05 GEMMs, flash attention, fused norms), activation checkpointing except for the last micro-batch.
`--impl reference`: the UNMODIFIED reference `Pipe` (single process, one worker thread and copy streams per device,
fairscale/nn/pipe/pipe.py:174-418) around the same architecture built from torch.nn modules; it needs every GPU visible
to one process, so it is started without torchrun.  Tokens/s is device-timed on the last stage (it finishes last).
Synthetic tokens, random-init weights.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
from torch import nn
from torch.nn import functional as F

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def balance_of(n_layers: int, stages: int):
    base, rem = divmod(n_layers, stages)
    return [base + (1 if i < rem else 0) for i in range(stages)]


class _RefEmbed(nn.Module):
    def __init__(self, vocab, d, seq):
        super().__init__()
        self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(seq, d)

    def forward(self, tokens):
        return self.wte(tokens) + self.wpe(torch.arange(tokens.shape[1], device=tokens.device))


class _RefBlock(nn.Module):
    def __init__(self, d, heads, ffn):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc1, self.fc2 = nn.Linear(d, ffn), nn.Linear(ffn, d)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, s, d))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


class _RefHead(nn.Module):
    def __init__(self, vocab, d):
        super().__init__()
        self.ln_f, self.out = nn.LayerNorm(d), nn.Linear(d, vocab, bias=False)

    def forward(self, x):
        return self.out(self.ln_f(x))


def run_reference(args):
    sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
    from fairscale.nn import Pipe  # the reference library, stock code path

    devices = [torch.device("cpu")] * args.stages if args.cpu else [torch.device("cuda", i) for i in range(args.stages)]
    dtype = torch.float32 if args.cpu else torch.bfloat16
    torch.manual_seed(0)
    layers = [_RefEmbed(args.vocab, args.d_model, args.seq)] + [_RefBlock(args.d_model, args.heads, args.ffn) for _ in range(args.layers)]
    layers.append(_RefHead(args.vocab, args.d_model))
    model = nn.Sequential(*layers).to(dtype)
    pipe = Pipe(model, balance_of(len(layers), args.stages), devices=devices, chunks=args.chunks, checkpoint="except_last")
    opt = torch.optim.Adam(pipe.parameters(), lr=1e-4, fused=not args.cpu)
    first, last = devices[0], devices[-1]
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, args.vocab, (args.batch, args.seq + 1), generator=g)
    x, y = toks[:, :-1].contiguous().to(first), toks[:, 1:].contiguous().to(last)

    def step():
        out = pipe(x)
        loss = F.cross_entropy(out.float().view(-1, out.shape[-1]), y.view(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    for _ in range(args.warmup):
        step()
    if args.cpu:
        import time

        t0 = time.time()
        for _ in range(args.steps):
            loss = step()
        ms = (time.time() - t0) * 1e3 / args.steps
    else:
        for d in devices:
            torch.cuda.synchronize(d)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.device(first):
            a.record()
        for _ in range(args.steps):
            loss = step()
        for d in devices:
            torch.cuda.synchronize(d)
        with torch.cuda.device(first):
            b.record()
            b.synchronize()
        ms = a.elapsed_time(b) / args.steps
    print(json.dumps({"benchmark": "pipe_lm", "impl": "reference", "stages": args.stages, "chunks": args.chunks, "layers": args.layers,
                      "ms_per_step": round(ms, 2), "tokens_per_s": round(args.batch * args.seq / ms * 1e3, 1), "loss": float(loss.detach())}))


def run_ours(args):
    from fairscale_b200.models.gpt import Block, Embedding, GPTConfig, Head
    from fairscale_b200.nn.pipe import AsyncPipe, LazyModule
    from fairscale_b200.optim import FusedAdam

    rank = int(os.environ.get("LOCAL_RANK", "0"))
    if "RANK" not in os.environ:
        os.environ.update(RANK="0", WORLD_SIZE="1", MASTER_ADDR="127.0.0.1", MASTER_PORT="29551")
    if args.cpu:
        dev, dtype = torch.device("cpu"), torch.float32
        dist.init_process_group("gloo")
    else:
        torch.cuda.set_device(rank)
        dev, dtype = torch.device("cuda", rank), torch.bfloat16
        dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    stages = min(args.stages, world)
    cfg = GPTConfig(args.vocab, args.d_model, args.heads, args.layers, args.ffn, args.seq)
    torch.manual_seed(0)
    # every rank builds only the layers of its own stage
    layers = [LazyModule(lambda: Embedding(cfg).to(dtype))] + [LazyModule(lambda: Block(cfg).to(dtype)) for _ in range(args.layers)]
    layers.append(LazyModule(lambda: Head(cfg).to(dtype)))
    pipe = AsyncPipe(layers, balance_of(len(layers), stages), chunks=args.chunks, checkpoint="except_last", input_device=dev)
    params = list(pipe.parameters())
    opt = (torch.optim.Adam(params, lr=1e-4) if args.cpu else FusedAdam(params, lr=1e-4)) if params else None
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, args.vocab, (args.batch, args.seq + 1), generator=g)
    x, y = toks[:, :-1].contiguous().to(dev), toks[:, 1:].contiguous().to(dev)
    last = stages - 1
    r = dist.get_rank()

    def step():
        out = pipe(x if r == 0 else None)
        loss = None
        if r == last:
            loss = F.cross_entropy(out.float().view(-1, out.shape[-1]), y.view(-1))
            loss.backward()
        pipe.back_helper(out if r < last else None)
        if opt is not None:
            opt.step()
            opt.zero_grad(set_to_none=True)
        return loss

    for _ in range(args.warmup):
        step()
    dist.barrier()
    if args.cpu:
        import time

        t0 = time.time()
        for _ in range(args.steps):
            loss = step()
        dist.barrier()
        ms = torch.tensor([(time.time() - t0) * 1e3 / args.steps])
    else:
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            loss = step()
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if r == last:
        print(json.dumps({"benchmark": "pipe_lm", "impl": "ours", "stages": stages, "chunks": args.chunks, "layers": args.layers,
                          "ms_per_step": round(float(ms), 2), "tokens_per_s": round(args.batch * args.seq / float(ms) * 1e3, 1),
                          "loss": float(loss.detach())}))
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=46, help="transformer blocks; with the embedding and the head: 48 pipeline layers")
    ap.add_argument("--d_model", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=256, help="global batch (sequences per step)")
    ap.add_argument("--chunks", type=int, default=32)
    ap.add_argument("--stages", type=int, default=8)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--cpu", action="store_true", help="gloo / CPU devices (functional check with tiny sizes)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
