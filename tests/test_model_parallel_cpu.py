"""Tensor-parallel layers on gloo ranks vs. their dense counterparts (same seed => same master weights)."""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn import model_parallel as mpu


def _groups(rank, world):
    mpu.initialize_model_parallel(2, pipeline_length=1, context_parallel_size=2)
    assert mpu.model_parallel_is_initialized()
    assert mpu.get_model_parallel_world_size() == 2
    assert mpu.get_context_parallel_world_size() == 2
    assert mpu.get_data_parallel_world_size() == world // 4
    assert mpu.get_model_parallel_rank() == rank % 2
    assert mpu.get_model_parallel_src_rank() == (rank // 2) * 2
    assert mpu.get_context_parallel_ranks() == ([0, 2] if rank in (0, 2) else [1, 3])
    assert mpu.get_pipeline_parallel_ranks() == [rank]
    mpu.destroy_model_parallel()
    assert not mpu.model_parallel_is_initialized()


def test_initialize_grid():
    spawn_ranks(_groups, 4, (), backend="gloo")


def _layers(rank, world):
    mpu.initialize_model_parallel(world)
    tp = mpu.get_model_parallel_world_size()
    torch.manual_seed(1234)
    x = torch.randn(5, 3, 16, requires_grad=True)

    # column parallel, gathered output == dense linear with the master weight
    torch.manual_seed(7)
    col = mpu.ColumnParallelLinear(16, 24, bias=True, gather_output=True, keep_master_weight_for_test=True)
    dense_w = col.master_weight.clone()
    y = col(x)
    ref = F.linear(x, dense_w)
    torch.testing.assert_close(y, ref, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(col.get_master_weight(), dense_w)
    y.sum().backward()
    torch.testing.assert_close(x.grad, torch.autograd.grad(F.linear(x, dense_w).sum(), x)[0], atol=1e-5, rtol=1e-5)

    # row parallel with scattered input
    torch.manual_seed(8)
    row = mpu.RowParallelLinear(16, 12, bias=True, input_is_parallel=False, keep_master_weight_for_test=True)
    with torch.no_grad():
        row.bias.fill_(0.5)
    y2 = row(x.detach())
    torch.testing.assert_close(y2, F.linear(x.detach(), row.master_weight) + 0.5, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(row.get_master_weight(), row.master_weight)

    # column (no gather) feeding row (parallel input): the Megatron MLP pattern
    torch.manual_seed(9)
    c2 = mpu.ColumnParallelLinear(16, 32, gather_output=False, keep_master_weight_for_test=True)
    r2 = mpu.RowParallelLinear(32, 16, input_is_parallel=True, keep_master_weight_for_test=True)
    h = r2(torch.relu(c2(x.detach())))
    ref_h = F.linear(torch.relu(F.linear(x.detach(), c2.master_weight)), r2.master_weight)
    torch.testing.assert_close(h, ref_h, atol=1e-5, rtol=1e-5)

    # embeddings
    torch.manual_seed(10)
    tok = torch.randint(0, 40, (4, 6))
    torch.manual_seed(11)
    ve = mpu.VocabParallelEmbedding(40, 8)
    torch.manual_seed(11)
    full = torch.empty(40, 8)
    torch.nn.init.xavier_normal_(full)
    torch.testing.assert_close(ve(tok), F.embedding(tok, full))
    torch.manual_seed(12)
    pe = mpu.ParallelEmbedding(40, 8)
    torch.manual_seed(12)
    full2 = torch.empty(40, 8)
    torch.nn.init.xavier_normal_(full2)
    torch.testing.assert_close(pe(tok), F.embedding(tok, full2))

    # vocab-parallel cross entropy == dense cross entropy
    torch.manual_seed(13)
    logits = torch.randn(4, 6, 40)
    target = torch.randint(0, 40, (4, 6))
    shard = logits.chunk(tp, dim=-1)[mpu.get_model_parallel_rank()].clone().requires_grad_()
    loss = mpu.vocab_parallel_cross_entropy(shard, target)
    dense = logits.clone().requires_grad_()
    ref_loss = F.cross_entropy(dense.view(-1, 40), target.view(-1), reduction="none").view(4, 6)
    torch.testing.assert_close(loss, ref_loss, atol=1e-5, rtol=1e-5)
    loss.sum().backward()
    ref_loss.sum().backward()
    torch.testing.assert_close(shard.grad, dense.grad.chunk(tp, dim=-1)[mpu.get_model_parallel_rank()], atol=1e-5, rtol=1e-5)

    # RNG tracker: the model-parallel stream differs across tp ranks, the default stream does not
    mpu.model_parallel_cuda_manual_seed(123)
    a = torch.rand(1)
    with mpu.get_cuda_rng_tracker().fork():
        b = torch.rand(1)
    ga = [torch.zeros(1) for _ in range(world)]
    gb = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(ga, a)
    dist.all_gather(gb, b)
    assert all(torch.equal(ga[0], t) for t in ga)
    assert not torch.equal(gb[0], gb[1])

    # RNG-aware checkpoint reproduces dropout
    lin = torch.nn.Linear(16, 16)
    def fn(t):
        with mpu.get_cuda_rng_tracker().fork():
            return F.dropout(lin(t), 0.5, training=True)
    xin = torch.randn(3, 16, requires_grad=True)
    out = mpu.checkpoint(fn, xin)
    out.sum().backward()
    assert xin.grad is not None and lin.weight.grad is not None


def test_layers_match_dense():
    spawn_ranks(_layers, 2, (), backend="gloo")


def test_rng_tracker_single_process():
    """Named RNG streams: a fork draws from its own stream and leaves the default one untouched, streams continue where
    they stopped, states can be saved and restored (on CPU the tracker drives the CPU generator)."""
    import pytest

    from fairscale_b200.nn.model_parallel.random import CudaRNGStatesTracker

    tr = CudaRNGStatesTracker()
    torch.manual_seed(1)
    tr.add("a", 100)
    tr.add("b", 200)
    with pytest.raises(Exception):
        tr.add("a", 300)  # the name is taken
    with pytest.raises(Exception):
        tr.add("c", 100)  # the seed is taken
    with pytest.raises(Exception):
        with tr.fork("missing"):
            pass
    torch.manual_seed(1)
    expected_default = torch.rand(4)
    torch.manual_seed(1)
    with tr.fork("a"):
        a1 = torch.rand(4)
    assert torch.equal(torch.rand(4), expected_default)  # the fork did not consume the default stream
    snapshot = tr.get_states()
    with tr.fork("a"):
        a2 = torch.rand(4)
    assert not torch.equal(a1, a2)  # the stream went on
    tr.set_states(snapshot)
    with tr.fork("a"):
        assert torch.equal(torch.rand(4), a2)  # restored: the same continuation
    torch.manual_seed(100)
    assert torch.equal(torch.rand(4), a1)  # stream "a" is the generator seeded with 100
    with tr.fork("b"):
        assert not torch.equal(torch.rand(4), a1)
    tr.reset()
    assert tr.get_states() == {}
