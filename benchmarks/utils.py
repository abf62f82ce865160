"""Shared argument parsing and helpers of the benchmark scripts (reference: benchmarks/utils.py:24-167)."""

import argparse
import os
import time

import torch
import torch.distributed as dist


def init_args(description: str = "benchmark") -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=description)
    p.add_argument("--use_synthetic_data", action="store_true", default=True, help="random token stream (the only offline option)")
    p.add_argument("--dry_run", action="store_true", help="tiny model, few batches, CPU allowed")
    p.add_argument("--model_name", default="lm", choices=["lm", "seq"])
    p.add_argument("--debug", action="store_true")
    p.add_argument("--max_batch", type=int, default=4, help="measured batches per rank (after one warm-up batch)")
    p.add_argument("--world_size", type=int, default=0, help="processes to spawn (0: every visible GPU, or 2 on CPU)")
    p.add_argument("--cpu", action="store_true", help="gloo on CPU")
    return p


def device_and_backend(args, rank: int):
    if args.cpu or not torch.cuda.is_available():
        return torch.device("cpu"), "gloo"
    torch.cuda.set_device(rank)
    return torch.device("cuda", rank), "nccl"


def init_dist(rank: int, world: int, backend: str, port: int = 29501) -> None:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(port))
    kw = {"device_id": torch.device("cuda", rank)} if backend == "nccl" else {}
    dist.init_process_group(backend, rank=rank, world_size=world, **kw)


def tiny_lm_config(cfg: dict) -> dict:
    out = dict(cfg)
    out.update({"vocab_size": 512, "ninp": 64, "nhid": 128, "nhead": 4, "num_decoder_layers": 2, "seq_len": min(cfg["seq_len"], 17)})
    return out


class WpsMeter:
    """Words per second from the second batch on (the first one pays allocator and autotune warm-up)."""

    def __init__(self) -> None:
        self.words = 0
        self.t0 = None

    def step(self, n_words: int, device: torch.device) -> None:
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        if self.t0 is None:
            self.t0 = time.perf_counter()
            return
        self.words += n_words

    def wps(self) -> float:
        return self.words / max(time.perf_counter() - self.t0, 1e-9) if self.t0 is not None else 0.0


def check_golden(wps: float, peak_mem: float, golden: dict, rank: int = 0) -> bool:
    ok = wps > golden["avg_wps"] - 3 * golden["std_dev_wps"]
    mem = golden.get("peak_mem_usage")
    if mem is not None and peak_mem > 0:
        bar = mem[rank] if isinstance(mem, (list, tuple)) else mem
        ok = ok and peak_mem < 1.1 * bar
    return ok
