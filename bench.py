#!/usr/bin/env python
"""Flagship benchmark: FSDP full-shard training of the 1.3B GPT (tokens/s, whole job).

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 8 --warmup 3
    python bench.py --impl reference ...        # the unmodified reference (baseline/_ref) on the same model/config

Config: 24 layers, d_model 2048, 16 heads, FFN 8192, vocab 50304, seq 2048, micro-batch 8 per GPU,
FSDP(reshard_after_forward, flatten_parameters, bf16 compute / fp32 master), checkpoint_wrapper per block,
fused Adam; synthetic uniform tokens, N(0, 0.02) weights; weak scaling (per-GPU work fixed).

Two timed regions of K steps each, both bracketed by barrier + synchronize and timed with CUDA events
(max over ranks): `value` has the batch resident on the device; `e2e` copies every step's tokens from pinned
host memory and reads the loss back to the host.  One JSON line is printed by rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch
import torch.distributed as dist

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

CFG = dict(vocab=50304, d_model=2048, n_heads=16, n_layers=24, ffn=8192, seq=2048, micro_batch=8)
CLOCK_QUERY = (
    "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
    "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
)


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=CFG["n_layers"], help="debug only: a run with fewer layers is not a valid benchmark")
    ap.add_argument("--micro-batch", type=int, default=CFG["micro_batch"])
    ap.add_argument("--seq", type=int, default=CFG["seq"])
    ap.add_argument("--breakdown", action="store_true",
                    help="also print per-step collective / exposed-wait times (CUDA events on the streams that run them)")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples for one GPU while the timed region runs (read only)."""

    def __init__(self, gpu_index: int):
        self.path = tempfile.mkstemp(suffix=".csv")[1]
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL,
            )
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        finally:
            try:
                os.remove(self.path)
            except OSError:
                pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def init_dist(n_gpus: int) -> tuple:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n_gpus:
        if world == 1 and n_gpus > 1:
            raise SystemExit("for --gpus N > 1 launch through torch.distributed.run with --nproc-per-node N")
    torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        if "MASTER_ADDR" in os.environ and "MASTER_PORT" in os.environ and world > 1:
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
        else:
            import socket

            with socket.socket() as s:
                s.bind(("127.0.0.1", 0))
                port = s.getsockname()[1]
            dist.init_process_group("nccl", rank=0, world_size=1, init_method=f"tcp://127.0.0.1:{port}")
    return rank, world, local_rank


def build_ours(args: argparse.Namespace, device: torch.device):
    from fairscale_b200.models.gpt import GPTConfig, build_fsdp_gpt
    from fairscale_b200.optim import FusedAdam

    cfg = GPTConfig(CFG["vocab"], CFG["d_model"], CFG["n_heads"], args.layers, CFG["ffn"], args.seq)
    torch.manual_seed(0)
    model = build_fsdp_gpt(cfg, device)
    opt = FusedAdam(model.parameters(), lr=1e-4, betas=(0.9, 0.95), eps=1e-8)
    # The Adam kernel also writes the bf16 compute shards.  FSB200_FUSED_RS_ADAM=1 runs the step of every block inside the
    # NVLink reduce-scatter of its gradient (one kernel per FSDP unit); measured slower than reduce-scatter + one full-width
    # Adam launch at 2 GPUs (206.4 vs 200.7 ms per step), so it is off unless asked for.
    model.attach_optimizer(opt, fuse_step_into_reduce_scatter=os.environ.get("FSB200_FUSED_RS_ADAM", "0") == "1")

    def step(tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        loss = model(tokens, targets)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    return step, cfg


def build_reference(args: argparse.Namespace, device: torch.device):
    sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
    sys.path.insert(0, os.path.join(REPO, "baseline"))
    import fairscale  # noqa: F401  (the unmodified reference install)
    from reference_gpt import build_reference_fsdp_gpt  # torch.nn model + fairscale FSDP / checkpoint_wrapper

    torch.manual_seed(0)
    model = build_reference_fsdp_gpt(CFG["vocab"], CFG["d_model"], CFG["n_heads"], args.layers, CFG["ffn"], args.seq, device)
    # the reference's fused Adam accepts only fp32/fp16 parameters and is not built by its default install
    params = list(model.parameters())
    world_is_one = dist.get_world_size() == 1
    for p in params:
        p.grad_dtype = None
    opt = torch.optim.Adam(params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, fused=True)

    def step(tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        logits = model(tokens)
        loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.size(-1)).float(), targets.view(-1))
        loss.backward()
        if world_is_one:
            # With a single rank the reference leaves compute-dtype (bf16) gradients on its fp32 master parameters
            # (its cast happens in the reduce-scatter callback, which only runs for sharded parameters), and no torch
            # optimizer accepts that; cast them as a user of the reference would have to.
            for p in params:
                if p.grad is not None and p.grad.dtype != p.dtype:
                    g = p.grad.to(p.dtype)
                    p.grad = None
                    p.grad = g
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    return step, None


def main() -> None:
    args = parse_args()
    if args.impl == "reference" and not os.path.isdir(os.path.join(REPO, "baseline", "_ref", "fairscale")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is missing (reference not installed)"}))
        return
    rank, world, local_rank = init_dist(args.gpus)
    device = torch.device("cuda", local_rank)
    try:
        step, cfg = (build_ours if args.impl == "ours" else build_reference)(args, device)
    except Exception as e:  # the reference may not run on this torch / GPU
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}))
            return
        raise

    B, S = args.micro_batch, args.seq
    gen = torch.Generator().manual_seed(1234 + rank)
    n_batches = max(args.steps, 1)
    host_tokens = [torch.randint(0, CFG["vocab"], (B, S + 1), generator=gen).pin_memory() for _ in range(n_batches)]
    dev_tokens = [t.to(device) for t in host_tokens]

    def run_resident(i: int) -> torch.Tensor:
        t = dev_tokens[i % n_batches]
        return step(t[:, :-1].contiguous(), t[:, 1:].contiguous())

    def run_e2e(i: int) -> float:
        t = host_tokens[i % n_batches].to(device, non_blocking=True)
        loss = step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
        return float(loss.item())  # device -> host read of the step's result, every step, before the next step starts

    try:
        for i in range(args.warmup):
            run_resident(i)
    except Exception as e:
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}))
            return
        raise

    from fairscale_b200.ops import _bind

    def timed(fn) -> tuple:
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        launches0 = _bind.launch_count()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0 = time.perf_counter()
        t0.record()
        last = None
        for i in range(args.steps):
            last = fn(i)
        t1.record()
        host_ms = (time.perf_counter() - h0) * 1e3  # time the host needed to enqueue the steps (it may run ahead of the device)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([t0.elapsed_time(t1), host_ms], device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms[0].item(), _bind.launch_count() - launches0, last, ms[1].item()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_resident, launches, last_loss, host_ms = timed(run_resident)
    clocks = sampler.stop() if sampler is not None else {}
    ms_e2e, _, last_e2e, _ = timed(run_e2e)

    breakdown = None
    if args.breakdown and args.impl == "ours":
        from fairscale_b200.utils import profiling

        tr = profiling.enable_comm_trace(True)
        timed(run_resident)
        summ = tr.summary()
        profiling.enable_comm_trace(False)
        breakdown = {k: {"calls_per_step": v["count"] / args.steps, "ms_per_step": round(v["total_ms"] / args.steps, 3)} for k, v in summ.items()}
    if args.impl == "ours":
        # a kernel whose bounded wait ran out leaves a code in the device status word: fail instead of reporting a number
        from fairscale_b200.utils.failure import check_device_status

        check_device_status(device)

    tokens_per_step = B * S * world
    value = tokens_per_step * args.steps / (ms_resident / 1e3)
    e2e_value = tokens_per_step * args.steps / (ms_e2e / 1e3)
    if rank == 0:
        peak_gb = torch.cuda.max_memory_allocated() / 2**30
        out = {
            "metric": "tokens/s (device, max over ranks)",
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_resident / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic uniform tokens, random-init N(0,0.02) weights",
            "impl": args.impl,
            "config": {
                "model": f"GPT {args.layers}L d{CFG['d_model']} h{CFG['n_heads']} ffn{CFG['ffn']} vocab{CFG['vocab']}",
                "global_batch": B * world,
                "seq_len": S,
                "parallelism": f"fsdp{world} full-shard, bf16 compute / fp32 master, checkpoint per block, fused Adam",
                "l2_policy": "per-step working set (>25 GB of parameters, optimizer state and activations) far exceeds the 126 MB L2",
            },
            "results": {
                "final_loss": float(last_loss.detach()) if last_loss is not None else None,
                "peak_mem_gb": round(peak_gb, 2),
                "host_enqueue_ms_per_step": round(host_ms / args.steps, 2),
            },
            "clocks": clocks,
            "e2e": {
                "value": e2e_value,
                "unit": "tokens/s",
                "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": B * (S + 1) * 8,
                "d2h_bytes_per_step": 4,
            },
            "gpu_launches": launches if args.impl == "ours" else 0,
        }
        if args.impl == "ours":
            from fairscale_b200.ops import attention

            out["results"]["attention_backend"] = attention.BACKEND
            if cfg is not None:
                out["results"]["model_tflops_per_gpu"] = round(cfg.flops_per_token(S) * B * S / (ms_resident / args.steps / 1e3) / 1e12, 1)
            if clocks.get("sm_mhz"):
                out["results"]["ms_x_mhz"] = round(ms_resident / args.steps * clocks["sm_mhz"], 0)  # clock-independent work figure
            if breakdown is not None:
                out["breakdown"] = breakdown
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
