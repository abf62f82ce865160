"""OffloadModel benchmark: the sequential LM (or a deep MLP) trained with its parameters in host memory
(reference driver: benchmarks/experimental/offload.py:92-435; golden numbers in golden_configs/lm_wikitext2.py).

    python benchmarks/experimental/offload.py [--model_name lm|seq] [--checkpoint_activation] [--num_microbatches 1] [--dry_run]
"""
import json
import os
import sys

import torch
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from benchmarks import utils  # noqa: E402
from benchmarks.datasets.wikitext2_data import get_dataloaders, get_synthetic_datasets  # noqa: E402
from benchmarks.golden_configs import lm_wikitext2  # noqa: E402
from fairscale_b200.experimental.nn import OffloadModel  # noqa: E402
from fairscale_b200.models.transformer_lm import TransformerLM  # noqa: E402


def main():
    p = utils.init_args("OffloadModel benchmark")
    p.add_argument("--checkpoint_activation", action="store_true", default=True)
    p.add_argument("--num_microbatches", type=int, default=1)
    p.add_argument("--slices", type=int, default=3)
    args = p.parse_args()
    device = torch.device("cuda", 0) if torch.cuda.is_available() and not args.cpu else torch.device("cpu")
    torch.manual_seed(0)
    if args.model_name == "lm":
        cfg = lm_wikitext2.Offload_Transformer.get_model_config()
        run_cfg = lm_wikitext2.Offload_Transformer.get_benchmark_config(args.checkpoint_activation)
        if args.dry_run:
            cfg = utils.tiny_lm_config(cfg)
        model = TransformerLM(cfg["vocab_size"], cfg["ninp"], cfg["nhead"], cfg["nhid"], cfg["dropout"], cfg["initrange"], cfg["num_decoder_layers"])
        train, _, _ = get_dataloaders(get_synthetic_datasets(cfg["vocab_size"], n=400000), run_cfg["batch_size"], cfg["seq_len"], max_batches=args.max_batch + 1)
        batches = [(b["input"], b["target"]) for b in train]
    else:
        cfg = lm_wikitext2.Offload_Sequential.get_model_config()
        run_cfg = lm_wikitext2.Offload_Sequential.get_benchmark_config()
        n_layers = 6 if args.dry_run else cfg["layers"]
        layers = [nn.Linear(cfg["inputs"], cfg["hidden"]), nn.ReLU()]
        for _ in range(n_layers):
            layers += [nn.Linear(cfg["hidden"], cfg["hidden"]), nn.ReLU()]
        layers.append(nn.Linear(cfg["hidden"], cfg["outputs"]))
        model = nn.Sequential(*layers)
        g = torch.Generator().manual_seed(0)
        batches = [(torch.randn(run_cfg["batch_size"], cfg["inputs"], generator=g), torch.randint(0, cfg["outputs"], (run_cfg["batch_size"],), generator=g))
                   for _ in range(args.max_batch + 1)]
    off = OffloadModel(model, device, torch.device("cpu"), num_slices=args.slices, checkpoint_activation=args.checkpoint_activation,
                       num_microbatches=args.num_microbatches)
    opt = torch.optim.SGD(off.parameters(), lr=run_cfg["lr"])
    crit = run_cfg["criterion"]
    meter = utils.WpsMeter()
    loss = torch.zeros(())
    for x, y in batches:
        opt.zero_grad()
        out = off(x.to(device) if x.is_floating_point() else x.to(device))
        loss = crit(out.float().view(-1, out.shape[-1]), y.to(out.device).view(-1))
        loss.backward()
        off.sync()
        opt.step()
        meter.step(x.numel() if args.model_name == "lm" else x.shape[0], device)
    res = {"benchmark": "offload", "model": args.model_name, "wps": round(meter.wps(), 1), "loss": float(loss.detach()), "dry_run": args.dry_run,
           "peak_mem_bytes": torch.cuda.max_memory_allocated(device) if device.type == "cuda" else 0}
    if args.model_name == "lm" and not args.dry_run:
        res["beats_reference_golden"] = utils.check_golden(meter.wps(), res["peak_mem_bytes"], lm_wikitext2.Offload_Transformer.get_golden_real_stats())
    print(json.dumps(res))


if __name__ == "__main__":
    main()
