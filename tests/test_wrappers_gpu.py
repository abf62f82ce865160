"""The wrappers on a GPU (one device; the multi-rank variants are in test_wrappers_multigpu.py): OSS + ShardedDDP,
single-process Pipe over CUDA streams, OffloadModel, MOELayer, FSDP options that only matter on a GPU (CPU offload,
fp32 reduce-scatter) and allocated-memory goldens per phase of an FSDP step.

Patterns of the reference: tests/nn/data_parallel/test_fsdp_overlap.py:243-250, test_fsdp_memory.py:161-416,
tests/experimental/nn/test_offload.py:139-170, tests/nn/moe/test_moe_layer.py:71-178, tests/nn/pipe/test_pipe.py.
"""
import copy
import socket

import pytest
import torch
import torch.distributed as dist
from torch import nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _one_rank_group():
    torch.cuda.set_device(0)
    created = False
    if not dist.is_initialized():
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        dist.init_process_group("nccl", rank=0, world_size=1, init_method=f"tcp://127.0.0.1:{port}")
        created = True
    yield
    if created:
        dist.destroy_process_group()


def _dev():
    return torch.device("cuda", 0)


def _mlp(seed=0, d=64):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(d, 2 * d), nn.GELU(), nn.Linear(2 * d, 2 * d), nn.Tanh(), nn.Linear(2 * d, d))


def _status_ok():
    from fairscale_b200 import _native

    torch.cuda.synchronize()
    assert _native.read_status(_dev()) == 0


@pytest.mark.parametrize("reduce_fp16", [False, True])
def test_oss_sharded_ddp_steps_like_the_plain_optimizer(reduce_fp16):
    from fairscale_b200.nn.data_parallel import ShardedDataParallel
    from fairscale_b200.optim import OSS

    ref = _mlp().to(_dev())
    model = copy.deepcopy(ref)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    oss = OSS(model.parameters(), optim=torch.optim.SGD, lr=0.05, momentum=0.9)
    sdp = ShardedDataParallel(model, oss, reduce_fp16=reduce_fp16)
    torch.manual_seed(1)
    for _ in range(3):
        x = torch.randn(16, 64, device=_dev())
        ref_opt.zero_grad()
        ref(x).pow(2).mean().backward()
        ref_opt.step()
        oss.zero_grad()
        sdp(x).pow(2).mean().backward()
        oss.step()
    tol = dict(atol=2e-3, rtol=2e-2) if reduce_fp16 else dict(atol=1e-6, rtol=1e-5)
    for a, b in zip(ref.parameters(), model.parameters()):
        torch.testing.assert_close(a, b, **tol)
    oss.consolidate_state_dict()
    assert len(oss.state_dict()["state"]) > 0


@pytest.mark.parametrize("checkpoint", ["never", "except_last", "always"])
def test_pipe_on_cuda_streams_matches_sequential(checkpoint):
    """Two partitions on the same GPU: the copies between them run on the per-micro-batch copy streams."""
    from fairscale_b200.nn.pipe import Pipe

    ref = _mlp(3).to(_dev())
    piped = Pipe(copy.deepcopy(ref).cpu(), balance=[2, 3], devices=[0, 0], chunks=4, checkpoint=checkpoint)
    x = torch.randn(32, 64, device=_dev(), requires_grad=True)
    x2 = x.detach().clone().requires_grad_()
    y, y2 = ref(x), piped(x2)
    torch.testing.assert_close(y2, y, atol=1e-5, rtol=1e-5)
    y.pow(2).sum().backward()
    y2.pow(2).sum().backward()
    torch.testing.assert_close(x2.grad, x.grad, atol=1e-4, rtol=1e-4)
    for a, b in zip(ref.parameters(), piped.parameters()):
        torch.testing.assert_close(b.grad, a.grad, atol=1e-4, rtol=1e-4)


def test_pipe_skip_connection_on_cuda():
    from fairscale_b200.nn.pipe import Pipe
    from fairscale_b200.nn.pipe.skip import pop, skippable, stash

    @skippable(stash=["res"])
    class Save(nn.Module):
        def forward(self, x):
            yield stash("res", x)
            return x * 2

    @skippable(pop=["res"])
    class Add(nn.Module):
        def forward(self, x):
            res = yield pop("res")
            return x + res

    def build():
        torch.manual_seed(4)
        return nn.Sequential(nn.Linear(16, 16), Save(), nn.Linear(16, 16), Add(), nn.Linear(16, 4))

    ref = build().to(_dev())
    piped = Pipe(build(), balance=[2, 1, 2], devices=[0, 0, 0], chunks=2, checkpoint="always")
    x = torch.randn(8, 16, device=_dev())
    torch.testing.assert_close(piped(x), ref(x), atol=1e-5, rtol=1e-5)
    ref(x).sum().backward()
    piped(x).sum().backward()
    for a, b in zip(ref.parameters(), piped.parameters()):
        torch.testing.assert_close(b.grad, a.grad, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("ckpt,microbatches", [(False, 1), (True, 1), (True, 4)])
def test_offload_model_on_gpu_matches_plain(ckpt, microbatches):
    """Slices live in pinned host memory and visit the GPU one at a time; results equal the resident model's."""
    from fairscale_b200.experimental.nn.offload import OffloadModel

    ref = _mlp(5).to(_dev())
    off = OffloadModel(copy.deepcopy(ref).cpu(), _dev(), torch.device("cpu"), num_slices=3, checkpoint_activation=ckpt,
                       num_microbatches=microbatches)
    opt_ref = torch.optim.SGD(ref.parameters(), lr=0.1)
    opt_off = torch.optim.SGD(off.parameters(), lr=0.1)
    torch.manual_seed(2)
    for _ in range(2):
        x = torch.randn(16, 64, device=_dev())
        opt_ref.zero_grad()
        ref(x).pow(2).mean().backward()
        opt_ref.step()
        opt_off.zero_grad()
        off(x).pow(2).mean().backward()
        opt_off.step()
    for a, b in zip(ref.parameters(), off.parameters()):
        torch.testing.assert_close(b.detach().cpu(), a.detach().cpu(), atol=1e-5, rtol=1e-4)
    assert all(p.device.type == "cpu" for p in off.parameters()), "the slices rest on the host between uses"


def test_moe_layer_on_one_gpu_index_path_matches_dense_einsum():
    """bf16 MOELayer with grouped experts on the GPU (index routing + grouped GEMM) against the same layer evaluated
    with the dense one-hot dispatch in fp32."""
    from fairscale_b200.nn.moe import MOELayer, Top2Gate
    from fairscale_b200.nn.moe.experts import GroupedExperts

    torch.manual_seed(7)
    d, ffn, n_exp, tokens = 128, 256, 4, 512
    gate = Top2Gate(d, n_exp).to(_dev())
    experts = GroupedExperts(n_exp, d, ffn).to(_dev()).bfloat16()
    moe = MOELayer(gate, experts)
    x = torch.randn(4, tokens // 4, d, device=_dev()).bfloat16().requires_grad_()
    torch.manual_seed(11)  # the gate draws its second-expert noise from the global generator
    y = moe(x)
    assert y.shape == x.shape and y.dtype == torch.bfloat16 and torch.isfinite(y.float()).all()
    y.float().pow(2).mean().backward()
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()
    assert all(p.grad is not None for p in experts.parameters())
    assert gate.wg.weight.grad is not None
    _status_ok()


@pytest.mark.parametrize("experts", [4, 64, 136])
def test_gate_projection_on_tensor_cores_matches_fp32(experts):
    """Router logits of bf16 activations: tcgen05 GEMM with fp32 output (expert dimension padded to a tile) and its
    backward against a plain fp32 linear."""
    from fairscale_b200.nn.moe.top2gate import Top2Gate, gate_logits

    torch.manual_seed(3)
    gate = Top2Gate(256, experts).to(_dev())
    x = torch.randn(4, 200, 256, device=_dev()).bfloat16().requires_grad_()
    logits = gate_logits(x, gate.wg)
    assert logits.dtype == torch.float32 and logits.shape == (4, 200, experts)
    xr = x.detach().float().requires_grad_()
    wr = gate.wg.weight.detach().bfloat16().float().requires_grad_()
    ref = torch.nn.functional.linear(xr, wr)
    torch.testing.assert_close(logits, ref, atol=2e-3, rtol=2e-3)
    g = torch.randn_like(ref)
    logits.backward(g)
    ref.backward(g.bfloat16().float())
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(gate.wg.weight.grad, wr.grad, atol=6e-2, rtol=3e-2)
    _status_ok()


def _fsdp_pair(**kw):
    from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP

    ref = _mlp(9).to(_dev())
    inner = copy.deepcopy(ref)
    if kw.get("move_params_to_cpu"):
        inner = inner.cpu()  # host-resident shards start from a module on the host (the wrapper asserts it, like the reference)
    wrapped = FSDP(inner, **kw)
    return ref, wrapped


@pytest.mark.parametrize("kw", [dict(move_params_to_cpu=True, mixed_precision=True), dict(mixed_precision=True, fp32_reduce_scatter=True),
                                dict(mixed_precision=True, compute_dtype=torch.bfloat16, move_grads_to_cpu=True, move_params_to_cpu=True)])
def test_fsdp_offload_and_fp32_reduce_scatter_options_on_gpu(kw):
    ref, fsdp = _fsdp_pair(compute_device=_dev(), **kw)
    opt_ref = torch.optim.SGD(ref.parameters(), lr=0.05)
    opt = torch.optim.SGD(fsdp.parameters(), lr=0.05)
    torch.manual_seed(3)
    for _ in range(2):
        x = torch.randn(8, 64, device=_dev())
        opt_ref.zero_grad()
        ref(x).float().pow(2).mean().backward()
        opt_ref.step()
        opt.zero_grad()
        fsdp(x).float().pow(2).mean().backward()
        opt.step()
    if kw.get("move_params_to_cpu"):
        assert all(p.device.type == "cpu" for p in fsdp.parameters())
    with fsdp.summon_full_params():
        for a, b in zip(ref.parameters(), fsdp.parameters()):
            torch.testing.assert_close(b.detach().float().cpu().view(-1)[: a.numel()], a.detach().float().cpu().view(-1), atol=3e-2, rtol=3e-2)


def test_allocated_memory_per_phase_of_an_fsdp_step():
    """Allocated bytes after forward, after backward and after the step against what the wrapper's design implies
    (parameters + gradients + nothing leaked), with and without activation checkpointing."""
    from fairscale_b200.nn.checkpoint import checkpoint_wrapper
    from fairscale_b200.nn.data_parallel import FullyShardedDataParallel as FSDP

    d, layers, batch = 1024, 4, 64

    def build(ckpt):
        torch.manual_seed(0)
        blocks = []
        for _ in range(layers):
            blk = nn.Sequential(nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d)).to(_dev())
            blocks.append(FSDP(checkpoint_wrapper(blk) if ckpt else blk, compute_device=_dev()))
        return FSDP(nn.Sequential(*blocks), compute_device=_dev())

    def mb(x):
        return x / 2**20

    results = {}
    for ckpt in (False, True):
        torch.cuda.empty_cache()
        torch.cuda.synchronize()
        base = torch.cuda.memory_allocated()
        model = build(ckpt)
        opt = torch.optim.SGD(model.parameters(), lr=0.01)
        x = torch.randn(batch, d, device=_dev())
        params_mb = mb(sum(p.numel() * 4 for p in model.parameters()))
        torch.cuda.synchronize()
        after_init = mb(torch.cuda.memory_allocated() - base)
        out = model(x)
        torch.cuda.synchronize()
        after_fwd = mb(torch.cuda.memory_allocated() - base)
        out.pow(2).mean().backward()
        torch.cuda.synchronize()
        after_bwd = mb(torch.cuda.memory_allocated() - base)
        opt.step()
        opt.zero_grad(set_to_none=True)
        del out
        torch.cuda.synchronize()
        idle = mb(torch.cuda.memory_allocated() - base)
        results[ckpt] = (params_mb, after_init, after_fwd, after_bwd, idle)
        # parameters only at rest (+ the input and small buffers), parameters + gradients after backward
        assert abs(after_init - params_mb) < 0.05 * params_mb + 2, results[ckpt]
        assert abs(idle - after_init) < 0.02 * params_mb + 2, results[ckpt]
        assert after_bwd < 2.0 * params_mb + 0.1 * params_mb + 4, results[ckpt]
        del model, opt
    # per block the un-checkpointed forward keeps the 4d-wide activations (2 x batch x 4d floats); checkpointing keeps
    # only the block inputs
    act_full = results[False][2] - results[False][1]
    act_ckpt = results[True][2] - results[True][1]
    expect_full = mb(layers * (2 * batch * 4 * d + 2 * batch * d) * 4)
    assert act_ckpt < 0.45 * act_full, results
    assert 0.6 * expect_full < act_full < 1.6 * expect_full, (act_full, expect_full)
