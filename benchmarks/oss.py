"""OSS / ShardedDDP benchmark against plain DDP (reference driver: benchmarks/oss.py:75-350): images/s, median / MAD
validation, optimizer-state consolidation every epoch.

    python benchmarks/oss.py --optim_type oss_sharded_ddp [--epochs 3] [--cpu] [--check_regression]
"""
import json
import os
import statistics
import sys
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn
from torch.nn.parallel import DistributedDataParallel as DDP
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks import utils  # noqa: E402
from benchmarks.datasets.mnist import setup_cached_mnist  # noqa: E402
from benchmarks.golden_configs import oss_mnist  # noqa: E402
from fairscale_b200.nn import ShardedDataParallel  # noqa: E402
from fairscale_b200.optim import OSS  # noqa: E402


def make_model():
    return nn.Sequential(nn.Conv2d(1, 32, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(32, 64, 3, padding=1), nn.ReLU(),
                         nn.MaxPool2d(2), nn.Flatten(), nn.Linear(64 * 7 * 7, 256), nn.ReLU(), nn.Linear(256, 10))


def train(rank, world, args, optim_type):
    device, backend = utils.device_and_backend(args, rank)
    utils.init_dist(rank, world, backend, port=29502)
    torch.manual_seed(0)
    model = make_model().to(device)
    data = setup_cached_mnist(2048 if args.cpu else 8192)
    loader = DataLoader(data, batch_size=args.batch_size, sampler=DistributedSampler(data, world, rank), drop_last=True)
    if optim_type == "vanilla":
        opt = torch.optim.RMSprop(model.parameters(), lr=1e-4, momentum=0.9)
        model = DDP(model, device_ids=[rank] if device.type == "cuda" else None)
    else:
        opt = OSS(model.parameters(), torch.optim.RMSprop, lr=1e-4, momentum=0.9)
        if optim_type == "oss_sharded_ddp":
            model = ShardedDataParallel(model, opt)
        else:
            model = DDP(model, device_ids=[rank] if device.type == "cuda" else None)
    loss_fn = nn.CrossEntropyLoss()
    speeds, final_loss = [], 0.0
    for epoch in range(args.epochs):
        n, t0 = 0, time.perf_counter()
        for x, y in loader:
            x, y = x.to(device), y.to(device)
            opt.zero_grad()
            loss = loss_fn(model(x), y)
            loss.backward()
            opt.step()
            n += x.shape[0] * world
            final_loss = float(loss)
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        speeds.append(n / (time.perf_counter() - t0))
        if isinstance(opt, OSS):
            opt.consolidate_state_dict()  # the checkpointing path is part of what is measured
            if rank == 0:
                opt.state_dict()
    if rank == 0:
        med = statistics.median(speeds)
        mad = statistics.median([abs(s - med) for s in speeds])
        res = {"benchmark": "oss", "optim_type": optim_type, "world_size": world, "img_per_s_median": round(med, 1), "mad": round(mad, 1),
               "final_loss": round(final_loss, 4),
               "peak_mem_mb": round(torch.cuda.max_memory_allocated(device) / 2**20, 1) if device.type == "cuda" else 0}
        if args.check_regression:
            res["beats_reference_golden"] = med + 8 * mad > oss_mnist.get_golden_real_stats()["reference_speed"]
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    p = utils.init_args("OSS / ShardedDDP benchmark")
    p.add_argument("--epochs", type=int, default=3)
    p.add_argument("--batch_size", type=int, default=256)
    p.add_argument("--optim_type", default="everyone", choices=["vanilla", "oss_ddp", "oss_sharded_ddp", "everyone"])
    p.add_argument("--check_regression", action="store_true")
    args = p.parse_args()
    world = args.world_size or (torch.cuda.device_count() if torch.cuda.is_available() and not args.cpu else 2)
    kinds = ["vanilla", "oss_ddp", "oss_sharded_ddp"] if args.optim_type == "everyone" else [args.optim_type]
    for kind in kinds:
        mp.spawn(train, args=(world, args, kind), nprocs=world, join=True)
