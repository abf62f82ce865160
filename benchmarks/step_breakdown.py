"""Per-kernel time of one training step of the flagship benchmark model (either arm), from the PyTorch profiler.

    python benchmarks/step_breakdown.py [--impl reference] [--layers 24] [--top 25]

Prints the plain (un-profiled) step time from CUDA events, the sum of GPU kernel time inside one profiled step and the
kernels ranked by total time.  Numbers taken under the profiler are for shares only; bench.py is the timing harness.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
from torch.profiler import ProfilerActivity, profile  # noqa: E402

import bench  # noqa: E402


def main() -> None:
    top = 25
    if "--top" in sys.argv:
        i = sys.argv.index("--top")
        top = int(sys.argv[i + 1])
        del sys.argv[i : i + 2]
    args = bench.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    bench.init_dist(1)
    built = (bench.build_ours if args.impl == "ours" else bench.build_reference)(args, dev)
    step = built[0] if isinstance(built, tuple) else built
    g = torch.Generator(device=dev).manual_seed(0)
    toks = torch.randint(0, bench.CFG["vocab"], (args.micro_batch, args.seq + 1), device=dev, generator=g)
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
    for _ in range(3):
        step(x, y)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    step(x, y)
    b.record()
    torch.cuda.synchronize()
    print(f"impl={args.impl} layers={args.layers}: plain step {a.elapsed_time(b):.1f} ms")
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        step(x, y)
        torch.cuda.synchronize()
    tot = {}
    for e in prof.events():
        if e.device_type == torch.autograd.DeviceType.CUDA:
            t = tot.setdefault(e.name[:70], [0.0, 0])
            t[0] += e.device_time
            t[1] += 1
    busy = sum(v[0] for v in tot.values())
    print(f"GPU kernel time in the profiled step: {busy / 1e3:.1f} ms")
    for k, v in sorted(tot.items(), key=lambda kv: -kv[1][0])[:top]:
        print(f"{v[0] / 1e3:9.2f} ms {v[1]:5d} x {v[0] / v[1]:8.1f} us  {k}")


if __name__ == "__main__":
    main()
