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

    # gather along the last dimension, written directly in the interleaved layout
    for shape in ((4, 8), (3, 5, 64), (257, 1024)):
        part = torch.randn(*shape, device=dev).bfloat16()
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        assert ws.can_all_gather_cols(torch.empty(*shape[:-1], shape[-1] * world, device=dev, dtype=torch.bfloat16), part)
        got = comm.all_gather_last_dim(part, None)
        assert torch.equal(got, torch.cat(parts, dim=-1))

    # reduce-scatter with fused scale + fp32 cast + accumulate, incl. implicit zero padding: the pull kernel, then the
    # copy-engine transport + local sum, which must give the same bits (same fp32 summation order)
    min_bytes = ws.DMA_MIN_BYTES
    for n, short in ((4096, 0), (1 << 18, 0), (1 << 14, 24)):
        full = (torch.randn(n * world - short, device=dev)).bfloat16()
        padded = torch.zeros(n * world, device=dev, dtype=torch.bfloat16)
        padded[: full.numel()] = full
        ref = torch.empty(n, device=dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(ref, padded.float())
        outs = {}
        for engine in ("kernel", "dma"):
            ws.reduce_scatter_engine, ws.DMA_MIN_BYTES = engine, 0
            out = torch.full((n,), 3.0, device=dev)
            ws.reduce_scatter(out, full, scale=0.5, accumulate=True)
            torch.testing.assert_close(out, 3.0 + 0.5 * ref, atol=2e-2, rtol=2e-2)
            out_b = torch.empty(n, device=dev, dtype=torch.bfloat16)
            comm.reduce_scatter_into(out_b, padded, None)
            torch.testing.assert_close(out_b.float(), ref, atol=6e-2, rtol=3e-2)
            outs[engine] = (out, out_b)
        assert torch.equal(outs["kernel"][0], outs["dma"][0]) and torch.equal(outs["kernel"][1], outs["dma"][1])
    ws.DMA_MIN_BYTES = min_bytes

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
    """FSDP over the NVLink data path (both all-gather engines, and with the optimizer step fused into the reduce-scatter)
    against FSDP over NCCL: same losses, same full parameters and the same Adam moments after three steps."""
    import os

    from fairscale_b200.models.gpt import GPTConfig, build_fsdp_gpt
    from fairscale_b200.optim import FusedAdam
    from fairscale_b200.parallel import comm, nvlink, symm
    from fairscale_b200.utils.failure import check_device_status

    dev = torch.device("cuda", rank)
    cfg = GPTConfig.tiny(vocab=1024, d_model=256, n_heads=2, n_layers=2, ffn=1024, max_seq=128)
    tokens = torch.randint(0, 1024, (2, 129), device=dev, generator=torch.Generator(device=dev).manual_seed(5 + rank))
    results = {}
    # keep_low_precision_grads=False: the unfused paths hand Adam an fp32 gradient shard, as the fused kernel does
    variants = [("nccl", "nccl", "kernel", False), ("nvlink-kernel", "fused", "kernel", False), ("nvlink-dma", "fused", "dma", False),
                ("nvlink-rs-adam", "fused", "dma", True)]
    for name, mode, engine, fuse_step in variants:
        os.environ["FSB200_COMM"] = mode
        torch.manual_seed(0)
        model = build_fsdp_gpt(cfg, dev, nvlink_heap=(mode == "fused"), keep_low_precision_grads=False, bucket_cap_mb=0)
        ws = symm.workspace_for(model.process_group)
        if ws is not None:
            ws.all_gather_engine = ws.reduce_scatter_engine = engine  # both collectives by pull kernels / by the copy engines
            ws.DMA_MIN_BYTES = 0
        opt = FusedAdam(model.parameters(), lr=1e-3, weight_decay=0.01)
        model.attach_optimizer(opt, fuse_step_into_reduce_scatter=fuse_step)
        comm.reset_counters()
        losses = []
        for _ in range(3):
            loss = model(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous())
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            losses.append(loss.item())
        check_device_status(dev)
        moments = torch.cat([opt.state[p]["exp_avg_sq"].view(-1) for p in model.parameters() if p in opt.state and "exp_avg_sq" in opt.state[p]])
        steps = sorted({int(opt.state[p]["step"]) for p in model.parameters() if p in opt.state and "step" in opt.state[p]})
        full = {k: v.float().clone() for k, v in model.state_dict().items()}
        results[name] = (losses, full, moments.clone(), steps)
        del model, opt
    assert symm.workspace_for(None) is not None
    ref_losses, ref_full, ref_moments, ref_steps = results["nccl"]
    assert ref_steps == [3]

    def rel(a, b):
        return float((a - b).norm() / b.norm().clamp_min(1e-12))

    def rms(t):
        return float(t.norm() / max(t.numel(), 1) ** 0.5)

    def same_training(name, ref_name, rel_tol, abs_allow, moment_tol):
        """Whole tensors by RMS, with an absolute allowance in units of the distance three Adam steps can move an element
        (3 * lr): Adam normalises the gradient, so last-bit differences of a gradient that is nearly zero come out as
        +-lr on single elements - all there is to see on parameters that start at zero."""
        losses, full, moments, steps = results[name]
        ref_l, ref_f, ref_m, _ = results[ref_name]
        assert steps == [3], (name, steps)
        torch.testing.assert_close(torch.tensor(losses), torch.tensor(ref_l), atol=2e-3, rtol=2e-3)
        assert full.keys() == ref_f.keys()
        for k in full:
            a, b = full[k], ref_f[k]
            if k.endswith("qkv_b"):
                # the softmax does not see a bias on the keys, so that third of the bias has a gradient of pure rounding
                # noise, whose sign Adam turns into +-lr per step: only the query and value thirds are comparable
                third = a.numel() // 3
                assert float((a[third : 2 * third] - b[third : 2 * third]).abs().max()) <= 2 * 3 * 1e-3 + 1e-6
                a, b = torch.cat([a[:third], a[2 * third :]]), torch.cat([b[:third], b[2 * third :]])
            assert rms(a - b) <= rel_tol * rms(b) + abs_allow * 3e-3, (name, k, rms(a - b), rms(b))
        assert rel(moments, ref_m) < moment_tol, (name, rel(moments, ref_m))

    # NCCL sums the bf16 gradients in bf16, the NVLink kernels in fp32
    for name in ("nvlink-kernel", "nvlink-dma", "nvlink-rs-adam"):
        same_training(name, "nccl", 2e-3, 0.05, 2e-2)
    # the two transports move the same bytes and sum in the same order: identical results
    for k in ref_full:
        assert torch.equal(results["nvlink-kernel"][1][k], results["nvlink-dma"][1][k]), k
    # the fused reduce-scatter + Adam kernel follows the formulas of reduce-scatter followed by the Adam kernel; the two are
    # compiled separately (different FMA contraction), so master weights differ in the last fp32 bit, a few compute-dtype
    # copies round the other way, and from the second step on the gradients differ in their noise
    same_training("nvlink-rs-adam", "nvlink-dma", 5e-4, 0.01, 5e-3)


def test_fsdp_over_nvlink_matches_nccl():
    spawn_ranks(_fsdp_worker, 2, (), backend="nccl", timeout=300)


def _rs_adam_worker(rank, world):
    """The fused reduce-scatter + Adam kernel against reduce-scatter followed by the multi-tensor Adam kernel."""
    from fairscale_b200.optim import FusedAdam
    from fairscale_b200.parallel import nvlink
    from fairscale_b200.utils.failure import check_device_status

    dev = torch.device("cuda", rank)
    ws = nvlink.enable(None, dev, staging_mb=16, heap_mb=64)
    n = 40960 + 8  # per-rank shard
    ws.enable_grad_windows(2 * (n * world + 64), count=2)
    torch.manual_seed(3)
    master = torch.randn(n, device=dev)
    a = torch.nn.Parameter(master.clone())
    b = torch.nn.Parameter(master.clone())
    copy_a = ws.alloc_tensor((n,), torch.bfloat16).zero_()
    copy_b = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    opt_a = FusedAdam([a], lr=1e-2, weight_decay=0.1, decoupled_weight_decay=True)
    opt_b = FusedAdam([b], lr=1e-2, weight_decay=0.1, decoupled_weight_decay=True)
    opt_a.param_copies[a] = copy_a
    opt_b.param_copies[b] = copy_b
    gsq = torch.zeros(1, device=dev)
    for step in range(3):
        torch.manual_seed(10 * step + rank)
        g = torch.randn(n * world, device=dev).bfloat16()
        window = ws.grad_window(n * world, torch.bfloat16, dev)
        window.copy_(g)
        assert opt_a.can_fuse_reduce_scatter(a) and ws.can_reduce_scatter_adam(window, a.data, a.data, a.data, copy_a)
        gsq.zero_()
        opt_a.reduce_scatter_step(a, ws, window, 1.0 / world, gnorm_sq=gsq)
        shard = torch.empty(n, device=dev)
        ws.reduce_scatter(shard, g, scale=1.0 / world)
        b.grad = shard
        opt_b.step()
        torch.testing.assert_close(gsq, shard.pow(2).sum().view(1), rtol=1e-4, atol=1e-6)
    check_device_status(dev)
    torch.testing.assert_close(a.data, b.data, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(opt_a.state[a]["exp_avg"], opt_b.state[b]["exp_avg"], atol=1e-7, rtol=1e-5)
    torch.testing.assert_close(opt_a.state[a]["exp_avg_sq"], opt_b.state[b]["exp_avg_sq"], atol=1e-9, rtol=1e-5)
    assert torch.equal(copy_a, copy_b) or (copy_a.float() - copy_b.float()).abs().max() < 1e-2
    assert opt_a.state[a]["step"] == opt_b.state[b]["step"] == 3
    dist.barrier()


def _wag_worker(rank, world):
    """Weight-gather GEMM: the flat parameter of a unit is all-gathered by the kernel that computes the unit's first
    product; both the gathered buffer and the product must be right, twice in a row (epochs / counters carry over)."""
    from fairscale_b200.parallel import fused_tp, nvlink
    from fairscale_b200.utils.failure import check_device_status

    dev = torch.device("cuda", rank)
    ws = nvlink.enable(None, dev, staging_mb=16, heap_mb=128)
    for (M, N, K, lead) in ((256, 512, 256, 0), (512, 1536, 512, 1024), (1024, 768, 1024, 8)):
        total = lead + N * K + N + 4096            # [leading small params | W | bias | trailing params]
        n = -(-total // (world * 8)) * 8            # elements per shard (multiple of 8)
        torch.manual_seed(11)
        flat = (torch.randn(n * world, device=dev) * 0.05).bfloat16()   # the same on every rank
        shard = ws.alloc_tensor((n,), torch.bfloat16)
        shard.copy_(flat[rank * n : (rank + 1) * n])
        torch.manual_seed(20 + rank)
        x = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
        bias = flat[lead + N * K : lead + N * K + N].clone()
        W = flat[lead : lead + N * K].view(N, K).float()
        ref = x.float() @ W.t() + bias.float()
        full = torch.empty(n * world, device=dev, dtype=torch.bfloat16)
        assert fused_tp.weight_gather_gemm_supported(ws, shard, full, lead, N, K)
        # copy CTAs inside the GEMM launch (default and a fixed count), then the copy-engine transport whose arrival
        # flags the GEMM waits on (one piece, then many small pieces)
        for engine, n_comm, piece in (("sm", None, None), ("sm", 4, None), ("dma", None, 2 << 20), ("dma", None, 64 << 10)):
            if piece is not None:
                fused_tp.WAG_PIECE_BYTES = piece
            full.fill_(float("nan"))
            y = fused_tp.weight_gather_gemm(ws, x, shard, full, lead, N, K, bias, n_comm=n_comm, engine=engine)
            torch.testing.assert_close(full, flat)
            torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=3e-2)
    check_device_status(dev)
    dist.barrier()


def test_weight_gather_gemm_fills_the_flat_parameter_and_computes_the_product():
    n = min(torch.cuda.device_count(), 8)
    spawn_ranks(_wag_worker, 2 if n < 4 else (4 if n < 8 else 8), (), backend="nccl", timeout=300)


def test_reduce_scatter_adam_kernel_matches_unfused():
    spawn_ranks(_rs_adam_worker, 2, (), backend="nccl", timeout=300)


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
        # copy CTAs inside the GEMM launch, then the copy-engine transport with arrival flags (one piece per block, then
        # 128-row pieces); twice each: epochs and monotonic counters must carry over
        for engine, piece in (("sm", None), ("dma", 4 << 20), ("dma", 128 * K * 2)):
            if piece is not None:
                fused_tp.AG_PIECE_BYTES = piece
            for _ in range(2):
                y, gathered = fused_tp.ag_gemm(ws, x, w, b, engine=engine)
                torch.testing.assert_close(gathered, full)
                torch.testing.assert_close(y.float(), full.float() @ w.float().t() + b.float(), atol=3e-2, rtol=3e-2)
            wkn = w.t().contiguous()  # [K, N] storage
            y2, _ = fused_tp.ag_gemm(ws, x, wkn, None, w_is_kn=True, engine=engine)
            torch.testing.assert_close(y2.float(), full.float() @ w.float().t(), atol=3e-2, rtol=3e-2)
        fused_tp.AG_PIECE_BYTES = 4 << 20

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


def _residency_worker(rank, world):
    """The persistent fused kernels and the in-place all-reduce next to a foreign kernel that holds 40 SMs for 20 ms on
    another stream: fewer SMs than CTAs must cost time only - right answers and a clean status word."""
    from fairscale_b200 import _native
    from fairscale_b200.fair_dev.testing.testing import gpu_occupy_sms
    from fairscale_b200.parallel import fused_tp, nvlink

    dev = torch.device("cuda", rank)
    ws = nvlink.enable(None, dev, staging_mb=16, heap_mb=256)
    torch.manual_seed(3 + rank)
    Mc, K, N = 1024, 1024, 2048
    M = Mc * world
    x = (torch.randn(Mc, K, device=dev) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
    full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(full, x)
    xa = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
    ref_rs = torch.empty(Mc, N, device=dev)
    dist.reduce_scatter_tensor(ref_rs, xa.float() @ w.float().t())
    t = (torch.randn(1 << 20, device=dev)).bfloat16()
    ref_ar = t.float().clone()
    dist.all_reduce(ref_ar)
    side = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    dist.barrier()
    for op in ("ag_gemm", "gemm_rs", "all_reduce"):
        gpu_occupy_sms(20.0, 40, side)
        if op == "ag_gemm":
            y, gathered = fused_tp.ag_gemm(ws, x, w, None)
            torch.testing.assert_close(gathered, full)
            torch.testing.assert_close(y.float(), full.float() @ w.float().t(), atol=3e-2, rtol=3e-2)
        elif op == "gemm_rs":
            out = fused_tp.gemm_rs(ws, xa, w, None)
            torch.testing.assert_close(out.float(), ref_rs, atol=6e-2, rtol=3e-2)
        else:
            buf = t.clone()
            assert ws.can_all_reduce(buf)
            ws.all_reduce(buf)
            torch.testing.assert_close(buf.float(), ref_ar, atol=6e-2, rtol=3e-2)
        torch.cuda.synchronize()
        assert _native.read_status(dev) == 0, op
    dist.barrier()


def test_persistent_kernels_survive_a_foreign_kernel_holding_sms():
    spawn_ranks(_residency_worker, 2, (), backend="nccl", timeout=300)


def _moe_layer_worker(rank, world):
    """MOELayer with grouped bf16 experts over the NVLink scatter / gather kernels (per-layer heap buffers, unclaimed rows
    zeroed by the scatter) against the same layer over NCCL all-to-all: outputs and every gradient, three iterations (the
    buffers are reused), then two forwards before the backwards (the layer must fall back to shared buffers + copies)."""
    import os

    from fairscale_b200.nn.moe import MOELayer, Top2Gate
    from fairscale_b200.nn.moe.experts import GroupedExperts
    from fairscale_b200.parallel import nvlink
    from fairscale_b200.utils.failure import check_device_status

    dev = torch.device("cuda", rank)
    nvlink.enable(None, dev, staging_mb=8, heap_mb=64)
    d, ffn, n_local, tokens = 128, 256, 2, 512
    torch.manual_seed(1)
    gate = Top2Gate(d, n_local * world).to(dev)
    torch.manual_seed(2 + rank)
    experts = GroupedExperts(n_local, d, ffn).to(dev).bfloat16()
    moe = MOELayer(gate, experts)

    def run(mode, x, seeds):
        os.environ["FSB200_COMM"] = mode
        moe.zero_grad()
        xs = [x.clone().requires_grad_() for _ in seeds]
        ys, aux = [], []
        for s, xi in zip(seeds, xs):
            torch.manual_seed(s)  # the gate draws its second-expert noise from the global generator
            ys.append(moe(xi))
            aux.append(moe.l_aux)
        for y, la in zip(ys, aux):
            (y.float().pow(2).mean() + la.float()).backward()
        grads = [p.grad.float().clone() for p in moe.parameters()]
        return [y.detach().float() for y in ys], [xi.grad.float() for xi in xs], grads

    def close(a, b):
        assert float((a - b).norm() / b.norm().clamp_min(1e-6)) < 2e-2

    for it in range(3):
        torch.manual_seed(100 + 10 * it + rank)
        x = torch.randn(4, tokens // 4, d, device=dev).bfloat16()
        for seeds in ([7 + it], [20 + it, 30 + it]):
            fused, ref = run("fused", x, seeds), run("nccl", x, seeds)
            for group_f, group_r in zip(fused, ref):
                for a, b in zip(group_f, group_r):
                    close(a, b)
    os.environ["FSB200_COMM"] = "fused"
    assert moe._heap_buffers.outstanding == 0 and not moe._heap_buffers.full
    check_device_status(dev)
    dist.barrier()


def test_moe_layer_over_nvlink_matches_all_to_all():
    spawn_ranks(_moe_layer_worker, 2, (), backend="nccl", timeout=300)


def test_fused_tp_kernels():
    n = min(torch.cuda.device_count(), 8)
    spawn_ranks(_fused_tp_worker, 2 if n < 4 else (4 if n < 8 else 8), (), backend="nccl", timeout=300)
