"""In-kernel NVLink collectives vs. NCCL on 2+ GPUs (one process per GPU, spawned by the test)."""
import pytest
import torch
import torch.distributed as dist

from fairscale_b200.fair_dev.testing.testing import spawn_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank, world):
    from fairscale_b200 import _native
    from fairscale_b200.parallel import comm, nvlink

    dev = torch.device("cuda", rank)
    ws = nvlink.enable(None, dev, staging_mb=64, heap_mb=64)
    torch.manual_seed(100 + rank)

    ws.barrier()
    # all-gather (staged and heap-resident inputs)
    for n in (8, 4096, 1 << 20):
        shard = torch.randn(n, device=dev).bfloat16()
        out = torch.empty(n * world, device=dev, dtype=torch.bfloat16)
        ref = torch.empty_like(out)
        dist.all_gather_into_tensor(ref, shard)
        comm.all_gather_into(out, shard, None)
        torch.testing.assert_close(out, ref)
    resident = ws.alloc_tensor((1 << 16,), torch.bfloat16)
    resident.copy_(torch.randn(1 << 16, device=dev))
    out = torch.empty((1 << 16) * world, device=dev, dtype=torch.bfloat16)
    ref = torch.empty_like(out)
    dist.all_gather_into_tensor(ref, resident)
    ws.all_gather(out, resident)
    torch.testing.assert_close(out, ref)

    # reduce-scatter with fused scale + fp32 cast + accumulate, incl. implicit zero padding
    for n, short in ((4096, 0), (1 << 18, 0), (1 << 14, 24)):
        full = (torch.randn(n * world - short, device=dev)).bfloat16()
        padded = torch.zeros(n * world, device=dev, dtype=torch.bfloat16)
        padded[: full.numel()] = full
        ref = torch.empty(n, device=dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(ref, padded.float())
        out = torch.full((n,), 3.0, device=dev)
        ws.reduce_scatter(out, full, scale=0.5, accumulate=True)
        torch.testing.assert_close(out, 3.0 + 0.5 * ref, atol=2e-2, rtol=2e-2)
        out_b = torch.empty(n, device=dev, dtype=torch.bfloat16)
        comm.reduce_scatter_into(out_b, padded, None)
        torch.testing.assert_close(out_b.float(), ref, atol=6e-2, rtol=3e-2)

    # all-reduce, several dtypes and a ragged size
    for dtype, n in ((torch.bfloat16, 1 << 20), (torch.float32, 1000003), (torch.bfloat16, 8), (torch.float16, 4100)):
        t = torch.randn(n, device=dev).to(dtype)
        ref = t.float().clone()
        dist.all_reduce(ref)
        comm.all_reduce(t, None)
        torch.testing.assert_close(t.float(), ref, atol=5e-2, rtol=3e-2)

    # all-to-all
    inp = torch.randn(world, 4, 256, device=dev).bfloat16()
    out = torch.empty_like(inp)
    ref = torch.empty_like(inp)
    dist.all_to_all_single(ref, inp)
    comm.all_to_all_single(out, inp, None)
    torch.testing.assert_close(out, ref)

    # MoE row scatter / gather over peer memory
    M, rows = 64, 16
    buf = ws.alloc_tensor((world * rows, M), torch.bfloat16)
    buf.zero_()
    x = torch.randn(rows, M, device=dev).bfloat16()
    dst_rank = (torch.arange(rows, device=dev, dtype=torch.int32) + rank) % world
    dst_row = (rank * rows + torch.arange(rows, device=dev, dtype=torch.int32)).int()
    dst_rank[0] = -1  # dropped token
    ws.moe_scatter_rows(buf, x, dst_rank, dst_row, None, 1)
    back = torch.empty(rows, M, device=dev, dtype=torch.bfloat16)
    w = torch.full((rows,), 2.0, device=dev)
    ws.moe_gather_rows(buf, back, dst_rank, dst_row, w, 1)
    expect = 2.0 * x.float()
    expect[0] = 0
    torch.testing.assert_close(back.float(), expect, atol=2e-2, rtol=2e-2)

    torch.cuda.synchronize()
    assert _native.read_status(dev) == 0
    dist.barrier()


def test_nvlink_collectives_match_nccl():
    n = min(torch.cuda.device_count(), 8)
    spawn_ranks(_worker, 2 if n < 4 else (4 if n < 8 else 8), (), backend="nccl", timeout=300)


def _fsdp_worker(rank, world):
    """FSDP over the NVLink collectives must produce the same losses as over NCCL."""
    import os

    from fairscale_b200.models.gpt import GPTConfig, build_fsdp_gpt
    from fairscale_b200.optim import FusedAdam
    from fairscale_b200.parallel import nvlink, symm

    dev = torch.device("cuda", rank)
    cfg = GPTConfig.tiny(vocab=1024, d_model=256, n_heads=2, n_layers=2, ffn=1024, max_seq=128)
    tokens = torch.randint(0, 1024, (2, 129), device=dev, generator=torch.Generator(device=dev).manual_seed(5 + rank))
    losses = {}
    for mode in ("nccl", "fused"):
        os.environ["FSB200_COMM"] = mode
        torch.manual_seed(0)
        model = build_fsdp_gpt(cfg, dev, nvlink_heap=(mode == "fused"))
        opt = FusedAdam(model.parameters(), lr=1e-3)
        model.attach_optimizer(opt)
        out = []
        for _ in range(3):
            loss = model(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous())
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            out.append(loss.item())
        losses[mode] = out
    assert symm.workspace_for(model.process_group) is not None
    torch.testing.assert_close(torch.tensor(losses["fused"]), torch.tensor(losses["nccl"]), atol=2e-2, rtol=2e-2)


def test_fsdp_over_nvlink_matches_nccl():
    spawn_ranks(_fsdp_worker, 2, (), backend="nccl", timeout=300)


def _fused_tp_worker(rank, world):
    """all-gather->GEMM and GEMM->reduce-scatter kernels vs an fp32 oracle built from NCCL collectives."""
    from fairscale_b200 import _native
    from fairscale_b200.parallel import fused_tp, nvlink

    dev = torch.device("cuda", rank)
    ws = nvlink.enable(None, dev, staging_mb=16, heap_mb=256)
    torch.manual_seed(7 + rank)
    for Mc, K, N in ((128, 64, 256), (256, 512, 384), (1024, 1024, 1536)):
        M = Mc * world
        x = (torch.randn(Mc, K, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
        b = torch.randn(N, device=dev).bfloat16()
        full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x)
        for _ in range(2):  # twice: epochs and monotonic counters must carry over
            y, gathered = fused_tp.ag_gemm(ws, x, w, b)
            torch.testing.assert_close(gathered, full)
            torch.testing.assert_close(y.float(), full.float() @ w.float().t() + b.float(), atol=3e-2, rtol=3e-2)
        wkn = w.t().contiguous()  # [K, N] storage
        y2, _ = fused_tp.ag_gemm(ws, x, wkn, None, w_is_kn=True)
        torch.testing.assert_close(y2.float(), full.float() @ w.float().t(), atol=3e-2, rtol=3e-2)

        xa = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
        partial = xa.float() @ w.float().t()
        ref = torch.empty(Mc, N, device=dev)
        dist.reduce_scatter_tensor(ref, partial)
        for _ in range(2):
            out = fused_tp.gemm_rs(ws, xa, w, b)
            torch.testing.assert_close(out.float(), ref + b.float(), atol=6e-2, rtol=3e-2)
    # through autograd: a column-parallel then a row-parallel linear, compared with the unfused path
    import os

    T, K, H = 256 * world, 512, 1024
    xs = (torch.randn(T // world, K, device=dev) * 0.5).bfloat16()
    w1 = (torch.randn(H, K, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(K, H, device=dev) * 0.05).bfloat16()
    res = {}
    for mode in ("fused", "nccl"):
        os.environ["FSB200_COMM"] = mode
        a, p1, p2 = xs.clone().requires_grad_(), w1.clone().requires_grad_(), w2.clone().requires_grad_()
        out = fused_tp.linear_reduce_scatter(torch.nn.functional.gelu(fused_tp.all_gather_linear(a, p1, None)), p2, None)
        out.float().pow(2).sum().backward()
        res[mode] = [out.detach().float(), a.grad.float(), p1.grad.float(), p2.grad.float()]
    os.environ["FSB200_COMM"] = "fused"
    # both paths round intermediates to bf16 at different points and the weight gradients sum over all tokens, so
    # single elements may differ by more than their own magnitude; compare in the Frobenius norm instead
    for f, n in zip(res["fused"], res["nccl"]):
        rel = (f - n).norm() / n.norm().clamp_min(1e-6)
        assert float(rel) < 2e-2, float(rel)
    torch.cuda.synchronize()
    assert _native.read_status(dev) == 0
    dist.barrier()


def test_fused_tp_kernels():
    n = min(torch.cuda.device_count(), 8)
    spawn_ranks(_fused_tp_worker, 2 if n < 4 else (4 if n < 8 else 8), (), backend="nccl", timeout=300)
