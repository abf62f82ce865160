"""BatchNorm vs torch SyncBatchNorm vs this library's SyncBatchNorm on [50, 2048, 7, 7] activations
(reference driver: benchmarks/experimental/sync_batchnorm.py:16-40).

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/experimental/sync_batchnorm.py
"""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from fairscale_b200.experimental.nn import SyncBatchNorm  # noqa: E402


def bench(bn, x, iters=20):
    for _ in range(3):
        bn(x).sum().backward()
    if x.is_cuda:
        torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(iters):
        bn(x).sum().backward()
    if x.is_cuda:
        torch.cuda.synchronize()
    return (time.perf_counter() - t0) / iters * 1e3


def main():
    cuda = torch.cuda.is_available()
    rank = int(os.environ.get("LOCAL_RANK", "0"))
    if cuda:
        torch.cuda.set_device(rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dist.init_process_group("nccl" if cuda else "gloo")
    dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
    shape = (50, 2048, 7, 7) if cuda else (8, 64, 7, 7)
    x = torch.randn(*shape, device=dev, requires_grad=True)
    res = {"benchmark": "sync_batchnorm", "world_size": dist.get_world_size(), "shape": shape}
    res["batchnorm_ms"] = round(bench(torch.nn.BatchNorm2d(shape[1]).to(dev), x), 3)
    if cuda:
        res["torch_syncbn_ms"] = round(bench(torch.nn.SyncBatchNorm(shape[1]).to(dev), x), 3)
    res["ours_syncbn_ms"] = round(bench(SyncBatchNorm(shape[1]).to(dev), x), 3)
    if dist.get_rank() == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
