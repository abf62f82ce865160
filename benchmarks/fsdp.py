"""FSDP language-model benchmark: one process per GPU, words/s and peak memory, optional check against the reference's
published regression numbers (reference driver: benchmarks/fsdp.py:45-403).

    python benchmarks/fsdp.py --use_synthetic_data [--enable_auto_wrap] [--full_fp16] [--benchmark_eval] [--dry_run --cpu]
"""
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks import utils  # noqa: E402
from benchmarks.datasets.wikitext2_data import get_dataloaders, get_synthetic_datasets  # noqa: E402
from benchmarks.golden_configs import lm_wikitext2  # noqa: E402
from fairscale_b200.models.transformer_lm import TransformerDecoderLayer, TransformerLM  # noqa: E402
from fairscale_b200.nn import FullyShardedDataParallel as FSDP  # noqa: E402
from fairscale_b200.nn import auto_wrap, enable_wrap, wrap  # noqa: E402


def build(cfg, args, device):
    model = TransformerLM(cfg["vocab_size"], cfg["ninp"], cfg["nhead"], cfg["nhid"], cfg["dropout"], cfg["initrange"], cfg["num_decoder_layers"])
    if args.full_fp16:
        model = model.to(torch.bfloat16)
    model = model.to(device)
    fsdp_kw = dict(flatten_parameters=True, mixed_precision=False, compute_device=device)
    if args.enable_auto_wrap:
        with enable_wrap(wrapper_cls=FSDP, **fsdp_kw):
            layers = [wrap(l) if isinstance(l, TransformerDecoderLayer) else l for l in model]
            return FSDP(nn.Sequential(*layers), **fsdp_kw)
    return FSDP(model, **fsdp_kw)


def run(rank, world, args):
    device, backend = utils.device_and_backend(args, rank)
    utils.init_dist(rank, world, backend)
    cfg = lm_wikitext2.FSDP.get_model_config()
    run_cfg = lm_wikitext2.FSDP.get_benchmark_config()
    if args.dry_run:
        cfg = utils.tiny_lm_config(cfg)
    torch.manual_seed(0)
    model = build(cfg, args, device)
    opt = torch.optim.Adam(model.parameters(), lr=run_cfg["lr"])
    train, _, _ = get_dataloaders(get_synthetic_datasets(cfg["vocab_size"], n=400000), run_cfg["batch_size"], cfg["seq_len"], rank, world,
                                  max_batches=args.max_batch + 1)
    meter = utils.WpsMeter()
    crit = run_cfg["criterion"]
    model.train(not args.benchmark_eval)
    loss = torch.zeros(())
    for batch in train:
        x, y = batch["input"].to(device), batch["target"].to(device)
        if args.benchmark_eval:
            with torch.no_grad():
                out = model(x)
        else:
            opt.zero_grad()
            out = model(x)
            loss = crit(out.float().view(-1, out.shape[-1]), y.view(-1))
            loss.backward()
            model.clip_grad_norm_(cfg["clip_value"])
            opt.step()
        meter.step(x.numel() * world, device)
    peak = torch.cuda.max_memory_allocated(device) if device.type == "cuda" else 0
    if rank == 0:
        res = {"benchmark": "fsdp", "world_size": world, "wps": round(meter.wps(), 1), "peak_mem_bytes": peak, "loss": float(loss),
               "auto_wrap": args.enable_auto_wrap, "dry_run": args.dry_run}
        if not args.dry_run and not args.benchmark_eval:
            res["beats_reference_golden"] = utils.check_golden(meter.wps(), peak, lm_wikitext2.FSDP.get_golden_synthetic_stats(), rank)
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    p = utils.init_args("FSDP LM benchmark")
    p.add_argument("--enable_auto_wrap", action="store_true")
    p.add_argument("--full_fp16", action="store_true", help="whole model in bf16 (the reduced-precision mode of this build)")
    p.add_argument("--benchmark_eval", action="store_true")
    args = p.parse_args()
    world = args.world_size or (torch.cuda.device_count() if torch.cuda.is_available() and not args.cpu else 2)
    mp.spawn(run, args=(world, args), nprocs=world, join=True)
