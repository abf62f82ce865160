"""The wrappers on 2 GPUs (one process per GPU over NCCL / the NVLink data path): OSS + ShardedDDP against DDP, AsyncPipe
across two devices, FSDP with host-resident shards, and the overlap of compute with the all-gather of the next unit.

Patterns of the reference: tests/nn/data_parallel/test_sharded_ddp_pytorch_parity.py:241-249,
tests/nn/data_parallel/test_fsdp_overlap.py:243-250, tests/nn/data_parallel/test_fsdp.py:336-357.
"""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _mlp(seed=0, d=64):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(d, 2 * d), nn.GELU(), nn.Linear(2 * d, 2 * d), nn.Tanh(), nn.Linear(2 * d, d))


def _oss_sdp_worker(rank, world, reduce_fp16, buffer_size, over_nvlink=False):
    from torch.nn.parallel import DistributedDataParallel as DDP

    from fairscale_b200.nn.data_parallel import ShardedDataParallel
    from fairscale_b200.optim import OSS

    dev = torch.device("cuda", rank)
    ws = None
    if over_nvlink:
        # gradient (buckets) reduced by the owner's pull kernel, updated parameters copied out of the owner's heap
        from fairscale_b200.parallel import nvlink

        ws = nvlink.enable(None, dev, staging_mb=8, heap_mb=64)
    ref = DDP(_mlp().to(dev), device_ids=[rank])
    model = _mlp().to(dev)
    ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-3)
    oss = OSS(model.parameters(), optim=torch.optim.Adam, lr=1e-3)
    sdp = ShardedDataParallel(model, oss, reduce_fp16=reduce_fp16, reduce_buffer_size=buffer_size)
    torch.manual_seed(10 + rank)
    for _ in range(4):
        x = torch.randn(16, 64, device=dev)
        ref_opt.zero_grad()
        ref(x).pow(2).mean().backward()
        ref_opt.step()
        oss.zero_grad()
        sdp(x).pow(2).mean().backward()
        oss.step()
    tol = dict(atol=3e-3, rtol=3e-2) if reduce_fp16 else dict(atol=1e-6, rtol=1e-4)
    for a, b in zip(ref.module.parameters(), model.parameters()):
        torch.testing.assert_close(b, a, **tol)
    if ws is not None:
        from fairscale_b200.utils.failure import check_device_status

        check_device_status(dev)
        assert ws.lanes[3].epoch >= 4 * 2, "reductions and broadcasts went over the NVLink lane"
        if buffer_size > 0:
            assert any(ws.offset_of(b.buffer) is not None for b in sdp._bucket_list), "gradient buckets live in the symmetric heap"
    dist.barrier()


@pytest.mark.parametrize("reduce_fp16,buffer_size", [(False, 2**23), (False, 0), (True, 2**23)])
def test_oss_sharded_ddp_matches_ddp_on_two_gpus(reduce_fp16, buffer_size):
    spawn_ranks(_oss_sdp_worker, 2, (reduce_fp16, buffer_size), backend="nccl", timeout=300)


@pytest.mark.parametrize("reduce_fp16,buffer_size", [(False, 2**23), (False, 0), (True, 0)])
def test_oss_sharded_ddp_over_nvlink_matches_ddp(reduce_fp16, buffer_size):
    spawn_ranks(_oss_sdp_worker, 2, (reduce_fp16, buffer_size, True), backend="nccl", timeout=300)


def _async_pipe_worker(rank, world):
    from fairscale_b200.nn.pipe import AsyncPipe

    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    ref = _mlp(2).to(dev)
    pipe = AsyncPipe(_mlp(2), balance=[3, 2], chunks=4, checkpoint="except_last", input_device=dev)
    pipe.transport.static_shapes = True
    torch.manual_seed(5)
    for step in range(2):
        x = torch.randn(16, 64, device=dev)
        out = pipe(x if rank == 0 else None)
        if rank == 1:
            torch.testing.assert_close(out, ref(x), atol=1e-5, rtol=1e-5)
            out.pow(2).sum().backward()
            pipe.back_helper()
        else:
            pipe.back_helper(out)
        ref.zero_grad()
        ref(x).pow(2).sum().backward()
        lo = [0, 3][rank]
        ref_params = [p for layer in list(ref)[lo : lo + [3, 2][rank]] for p in layer.parameters()]
        for a, b in zip(pipe.partition.parameters(), ref_params):
            torch.testing.assert_close(a.grad, b.grad, atol=1e-4, rtol=1e-4)
        pipe.partition.zero_grad()
    # second step: every (peer, micro-batch) contract exists, so only the slot-less chunk-count message had a header
    assert pipe.transport.headers_received <= 2 + 4 + 4
    dist.barrier()


def test_async_pipe_on_two_gpus_matches_sequential():
    spawn_ranks(_async_pipe_worker, 2, (), backend="nccl", timeout=300)


def _fsdp_offload_worker(rank, world):
    from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP

    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    ref = _mlp(4).to(dev)
    # host-resident shards start from a module on the host (the wrapper asserts it, like the reference)
    fsdp = FSDP(copy.deepcopy(ref).cpu(), mixed_precision=True, compute_dtype=torch.bfloat16, move_params_to_cpu=True, compute_device=dev)
    opt = torch.optim.SGD(fsdp.parameters(), lr=0.05)
    opt_ref = torch.optim.SGD(ref.parameters(), lr=0.05)
    torch.manual_seed(7)  # the same data on both ranks: the averaged gradient equals the local one
    for _ in range(2):
        x = torch.randn(8, 64, device=dev)
        opt_ref.zero_grad()
        ref(x).float().pow(2).mean().backward()
        opt_ref.step()
        opt.zero_grad()
        fsdp(x).float().pow(2).mean().backward()
        opt.step()
    assert all(p.device.type == "cpu" for p in fsdp.parameters()), "between steps the shards rest on the host"
    sd = fsdp.state_dict()
    for (k, a), b in zip(ref.state_dict().items(), sd.values()):
        torch.testing.assert_close(b.float().cpu(), a.float().cpu(), atol=3e-2, rtol=3e-2)
    dist.barrier()


def test_fsdp_with_host_resident_shards_on_two_gpus():
    spawn_ranks(_fsdp_offload_worker, 2, (), backend="nccl", timeout=300)


def _overlap_worker(rank, world, mode):
    """Every FSDP unit computes for 10 ms (delay kernel) and every all-gather is slowed by 10 ms on the all-gather
    stream.  Without overlap a forward over 5 units costs ~100 ms; with the next unit's gather prefetched behind the
    current unit's compute only the first gather is exposed."""
    import os

    from fairscale_b200.fair_dev.testing.testing import gpu_delay
    from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP
    from fairscale_b200.parallel import comm, nvlink

    os.environ["FSB200_COMM"] = mode
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    if mode == "fused":
        nvlink.enable(None, dev, staging_mb=16, heap_mb=16)

    class Slow(nn.Module):
        def __init__(self):
            super().__init__()
            self.w = nn.Parameter(torch.ones(4096))

        def forward(self, x):
            gpu_delay(10.0)
            return x * self.w.mean()

    def build():
        return FSDP(nn.Sequential(*[FSDP(Slow().to(dev), compute_device=dev) for _ in range(5)]), compute_device=dev)

    def timed(model, n=3):
        x = torch.ones(4, 4096, device=dev)
        for _ in range(2):  # the first pass records the execution order that prefetching follows
            model(x).sum().backward()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        with torch.no_grad():
            for _ in range(n):
                model(x)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    compute_only = timed(build())
    real = comm.all_gather_into

    def slowed(out, shard, group=None, async_op=False):
        gpu_delay(10.0)  # lands on whatever stream issues the gather: the all-gather stream
        return real(out, shard, group=group, async_op=async_op)

    comm.all_gather_into = slowed
    try:
        both = timed(build())
    finally:
        comm.all_gather_into = real
    assert 45.0 < compute_only < 80.0, compute_only
    # serial would be compute_only + 5 x 10 ms; the reference's criterion: (compute + all_gather) > 1.1 x both
    assert compute_only + 50.0 > 1.1 * both, (compute_only, both)
    assert both < compute_only + 25.0, (compute_only, both)
    dist.barrier()


@pytest.mark.parametrize("mode", ["nccl", "fused"])
def test_all_gather_of_the_next_unit_overlaps_compute(mode):
    spawn_ranks(_overlap_worker, 2, (mode,), backend="nccl", timeout=300)
