"""Single-process Pipe benchmark of the sequential LM over the visible GPUs (reference driver: benchmarks/pipe.py:64-314).

    python benchmarks/pipe.py [--chunks 4] [--checkpoint except_last] [--dry_run]
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks import utils  # noqa: E402
from benchmarks.datasets.wikitext2_data import get_dataloaders, get_synthetic_datasets  # noqa: E402
from benchmarks.golden_configs import lm_wikitext2  # noqa: E402
from fairscale_b200.models.transformer_lm import TransformerLM  # noqa: E402
from fairscale_b200.nn import Pipe  # noqa: E402


def generate_balance(n_devices: int, n_layers: int):
    base, rem = divmod(n_layers, n_devices)
    return [base + (1 if i < rem else 0) for i in range(n_devices)]


def main():
    p = utils.init_args("Pipe LM benchmark")
    p.add_argument("--chunks", type=int, default=1)
    p.add_argument("--checkpoint", default="except_last", choices=["always", "except_last", "never"])
    args = p.parse_args()
    cfg = lm_wikitext2.Pipe.get_model_config()
    run_cfg = lm_wikitext2.Pipe.get_benchmark_config()
    if args.dry_run:
        cfg = utils.tiny_lm_config(cfg)
    n_gpu = torch.cuda.device_count() if torch.cuda.is_available() and not args.cpu else 0
    n_dev = max(1, min(n_gpu, 4))
    devices = [torch.device("cuda", i) for i in range(n_dev)] if n_gpu else [torch.device("cpu")] * 2
    torch.manual_seed(0)
    model = TransformerLM(cfg["vocab_size"], cfg["ninp"], cfg["nhead"], cfg["nhid"], cfg["dropout"], cfg["initrange"], cfg["num_decoder_layers"])
    pipe = Pipe(model, generate_balance(len(devices), len(model)), devices=devices, chunks=args.chunks, checkpoint=args.checkpoint)
    opt = torch.optim.Adam(pipe.parameters(), lr=run_cfg["lr"])
    train, _, _ = get_dataloaders(get_synthetic_datasets(cfg["vocab_size"], n=400000), run_cfg["batch_size"], cfg["seq_len"], max_batches=args.max_batch + 1)
    meter = utils.WpsMeter()
    crit = run_cfg["criterion"]
    first, last = devices[0], devices[-1]
    loss = torch.zeros(())
    for batch in train:
        x, y = batch["input"].to(first), batch["target"].to(last)
        opt.zero_grad()
        out = pipe(x)
        loss = crit(out.float().view(-1, out.shape[-1]), y.view(-1))
        loss.backward()
        torch.nn.utils.clip_grad_value_(pipe.parameters(), cfg["clip_value"])
        opt.step()
        meter.step(x.numel(), last)
    peaks = [torch.cuda.max_memory_allocated(d) for d in devices] if n_gpu else []
    res = {"benchmark": "pipe", "devices": len(devices), "chunks": args.chunks, "wps": round(meter.wps(), 1), "peak_mem_bytes": peaks,
           "loss": float(loss), "dry_run": args.dry_run}
    if not args.dry_run:
        g = lm_wikitext2.Pipe.get_golden_real_stats()
        res["beats_reference_golden"] = meter.wps() > g["avg_wps"] - 3 * g["std_dev_wps"]
    print(json.dumps(res))


if __name__ == "__main__":
    main()
