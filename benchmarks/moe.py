"""Mixture-of-experts LM benchmark: DDP for the dense parts, experts sharded over the ranks with all-to-all dispatch
(reference driver: benchmarks/moe.py:28-130; it publishes no golden numbers).

    python benchmarks/moe.py [--dry_run --cpu]
"""
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks import utils  # noqa: E402
from benchmarks.datasets.wikitext2_data import get_dataloaders, get_synthetic_datasets  # noqa: E402
from benchmarks.golden_configs import lm_wikitext2  # noqa: E402
from fairscale_b200.models.transformer_lm import TransformerLM  # noqa: E402


def run(rank, world, args):
    device, backend = utils.device_and_backend(args, rank)
    utils.init_dist(rank, world, backend, port=29503)
    cfg = lm_wikitext2.MOE.get_model_config()
    run_cfg = lm_wikitext2.MOE.get_benchmark_config()
    if args.dry_run:
        cfg = utils.tiny_lm_config(cfg)
        run_cfg["batch_size"] = 4
    torch.manual_seed(0)
    model = TransformerLM(cfg["vocab_size"], cfg["ninp"], cfg["nhead"], cfg["nhid"], cfg["dropout"], cfg["initrange"],
                          cfg["num_decoder_layers"], is_moe=True, num_local_experts=cfg["num_local_experts"]).to(device)
    for n, p in model.named_parameters():  # expert weights differ per rank and must not be all-reduced by DDP
        if ".experts." in n:
            p.expert = True  # type: ignore[attr-defined]
    DDP._set_params_and_buffers_to_ignore_for_model(model, [n for n, _ in model.named_parameters() if ".experts." in n])
    ddp = DDP(model, device_ids=[rank] if device.type == "cuda" else None)
    opt = torch.optim.Adam(model.parameters(), lr=run_cfg["lr"])
    seq = cfg["seq_len"] - 1
    train, _, _ = get_dataloaders(get_synthetic_datasets(cfg["vocab_size"], n=400000), run_cfg["batch_size"], seq, rank, world, max_batches=args.max_batch + 1)
    meter = utils.WpsMeter()
    crit = run_cfg["criterion"]
    loss = torch.zeros(())
    for batch in train:
        x, y = batch["input"].to(device), batch["target"].to(device)
        opt.zero_grad()
        out = ddp(x)
        loss = crit(out.float().view(-1, out.shape[-1]), y.view(-1))
        loss.backward()
        opt.step()
        meter.step(x.numel() * world, device)
    if rank == 0:
        print(json.dumps({"benchmark": "moe", "world_size": world, "wps": round(meter.wps(), 1), "loss": float(loss), "dry_run": args.dry_run,
                          "peak_mem_bytes": torch.cuda.max_memory_allocated(device) if device.type == "cuda" else 0}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    args = utils.init_args("MoE LM benchmark").parse_args()
    world = args.world_size or (torch.cuda.device_count() if torch.cuda.is_available() and not args.cpu else 2)
    mp.spawn(run, args=(world, args), nprocs=world, join=True)
