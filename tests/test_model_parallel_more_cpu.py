"""Tensor parallelism on gloo ranks, piece by piece (cases of the reference's tests/nn/model_parallel/test_initialize.py,
test_layers.py, test_random.py, test_cross_entropy.py): grids of every shape that fits the world, guards of the accessors, the
four region mappings forward and backward, sliced initialisation with strides, gradients of the parallel layers against the
dense formulas, embeddings forward and backward, the loss on shards against the dense loss, the two random streams and the
checkpoint that replays them."""
import pytest
import torch
import torch.distributed as dist
import torch.nn.functional as F

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn import model_parallel as mpu
from fairscale_b200.nn.model_parallel import layers as tp_layers
from fairscale_b200.nn.model_parallel.mappings import (
    copy_to_model_parallel_region,
    gather_from_model_parallel_region,
    reduce_from_model_parallel_region,
    scatter_to_model_parallel_region,
)
from fairscale_b200.nn.model_parallel.utils import VocabUtility, divide_and_check_no_remainder, ensure_divisibility, split_tensor_along_last_dim


# ------------------------------------------------------------------------------------------------ helpers without ranks
def test_divisibility_helpers_and_vocabulary_ranges():
    assert divide_and_check_no_remainder(12, 4) == 3
    ensure_divisibility(12, 6)
    with pytest.raises(AssertionError, match="not divisible"):
        divide_and_check_no_remainder(12, 5)
    x = torch.arange(24.0).view(2, 12)
    views = split_tensor_along_last_dim(x, 3)
    assert [v.shape for v in views] == [(2, 4)] * 3 and not views[1].is_contiguous() and torch.equal(views[2], x[:, 8:])
    copies = split_tensor_along_last_dim(x, 3, contiguous_split_chunks=True)
    assert all(c.is_contiguous() for c in copies) and torch.equal(copies[1], views[1])
    with pytest.raises(AssertionError):
        split_tensor_along_last_dim(x, 5)
    assert VocabUtility.vocab_range_from_global_vocab_size(48, 2, 4) == (24, 36)
    assert VocabUtility.vocab_range_from_per_partition_vocab_size(10, 3, 8) == (30, 40)
    with pytest.raises(AssertionError):
        VocabUtility.vocab_range_from_global_vocab_size(50, 0, 4)


# ------------------------------------------------------------------------------------------------ grids
def _grid(rank, world, mp, pipeline, context):
    assert not mpu.model_parallel_is_initialized()
    with pytest.raises(AssertionError):
        mpu.get_model_parallel_group()
    with pytest.raises(AssertionError):
        mpu.get_data_parallel_group()
    mpu.initialize_model_parallel(mp, pipeline_length=pipeline, context_parallel_size=context)
    mp_eff = min(mp, world)
    dp = world // (mp_eff * pipeline * context)
    assert mpu.model_parallel_is_initialized()
    assert mpu.get_model_parallel_world_size() == mp_eff == dist.get_world_size(mpu.get_model_parallel_group())
    assert mpu.get_data_parallel_world_size() == dp == dist.get_world_size(mpu.get_data_parallel_group())
    assert mpu.get_context_parallel_world_size() == context and len(mpu.get_pipeline_parallel_ranks()) == pipeline
    # model-parallel ranks are consecutive; the source rank is the first of the group
    assert mpu.get_model_parallel_rank() == rank % mp_eff == dist.get_rank(mpu.get_model_parallel_group())
    assert mpu.get_model_parallel_src_rank() == rank - rank % mp_eff
    assert mpu.get_data_parallel_rank() == dist.get_rank(mpu.get_data_parallel_group())
    assert rank in mpu.get_data_parallel_ranks() and rank in mpu.get_pipeline_parallel_ranks() and rank in mpu.get_context_parallel_ranks()
    assert mpu.get_context_parallel_rank() == mpu.get_context_parallel_ranks().index(rank)
    # every rank is in exactly one group per axis, and the groups of one axis tile the world
    for ranks in (mpu.get_data_parallel_ranks(), mpu.get_pipeline_parallel_ranks(), mpu.get_context_parallel_ranks()):
        mine = torch.zeros(world)
        mine[ranks] = 1.0
        dist.all_reduce(mine)
        assert torch.equal(mine, torch.full((world,), float(len(ranks))))
    # a collective on each group sees the right number of members
    for group, size in ((mpu.get_model_parallel_group(), mp_eff), (mpu.get_data_parallel_group(), dp), (mpu.get_pipeline_parallel_group(), pipeline),
                        (mpu.get_context_parallel_group(), context)):
        one = torch.ones(1)
        dist.all_reduce(one, group=group)
        assert int(one) == size
    with pytest.raises(AssertionError, match="already initialized"):
        mpu.initialize_model_parallel(mp)
    mpu.destroy_model_parallel()
    assert not mpu.model_parallel_is_initialized()
    mpu.initialize_model_parallel(1)  # and it can be set up again with another shape
    assert mpu.get_model_parallel_world_size() == 1 and mpu.get_data_parallel_world_size() == world
    mpu.destroy_model_parallel()


@pytest.mark.parametrize("mp,pipeline,context", [(1, 1, 1), (2, 1, 1), (4, 1, 1), (2, 2, 1), (1, 4, 1), (1, 2, 2), (8, 1, 1)])
def test_grids_of_every_shape(mp, pipeline, context):
    spawn_ranks(_grid, 4, (mp, pipeline, context), backend="gloo")


def _bad_grid(rank, world):
    with pytest.raises(AssertionError):
        mpu.initialize_model_parallel(3)  # does not divide four ranks
    with pytest.raises(AssertionError):
        mpu.initialize_model_parallel(2, pipeline_length=4)
    assert not mpu.model_parallel_is_initialized()


def test_grids_that_do_not_fit_are_refused():
    spawn_ranks(_bad_grid, 4, (), backend="gloo")


# ------------------------------------------------------------------------------------------------ mappings
def _mappings(rank, world):
    mpu.initialize_model_parallel(world)
    base = torch.arange(12.0).view(2, 6) + 100 * rank

    x = base.clone().requires_grad_()
    y = copy_to_model_parallel_region(x)          # identity forward, sum of the ranks' gradients backward
    assert torch.equal(y, x)
    (y * (rank + 1)).sum().backward()
    assert torch.equal(x.grad, torch.full_like(x, float(sum(range(1, world + 1)))))

    x = base.clone().requires_grad_()
    y = reduce_from_model_parallel_region(x)      # sum forward, identity backward
    assert torch.equal(y, sum(torch.arange(12.0).view(2, 6) + 100 * r for r in range(world)))
    (y * (rank + 1)).sum().backward()
    assert torch.equal(x.grad, torch.full_like(x, float(rank + 1)))

    x = base.clone().requires_grad_()
    y = scatter_to_model_parallel_region(x)       # own slice of the last dimension forward, gather backward
    width = 6 // world
    assert torch.equal(y, x[:, rank * width:(rank + 1) * width])
    (y * (rank + 1)).sum().backward()
    want = torch.cat([torch.full((2, width), float(r + 1)) for r in range(world)], dim=-1)
    assert torch.equal(x.grad, want)

    x = base.clone().requires_grad_()
    y = gather_from_model_parallel_region(x)      # concatenation along the last dimension forward, own slice backward
    assert y.shape == (2, 6 * world) and y.is_contiguous()
    assert torch.equal(y, torch.cat([torch.arange(12.0).view(2, 6) + 100 * r for r in range(world)], dim=-1))
    weights = torch.arange(float(6 * world))
    (y * weights).sum().backward()
    assert torch.equal(x.grad, weights[rank * 6:(rank + 1) * 6].expand(2, 6))
    # three dimensions, as activations have
    z = torch.randn(3, 4, 5)
    g = gather_from_model_parallel_region(z)
    assert g.shape == (3, 4, 5 * world) and torch.equal(g[..., rank * 5:(rank + 1) * 5], z)
    mpu.destroy_model_parallel()

    # with a single model-parallel rank all four are the identity and cost no communication
    mpu.initialize_model_parallel(1)
    for fn in (copy_to_model_parallel_region, reduce_from_model_parallel_region, scatter_to_model_parallel_region, gather_from_model_parallel_region):
        x = base.clone().requires_grad_()
        y = fn(x)
        assert torch.equal(y, x)
        y.sum().backward()
        assert torch.equal(x.grad, torch.ones_like(x))
    mpu.destroy_model_parallel()


@pytest.mark.parametrize("world", [2, 3])
def test_region_mappings_forward_and_backward(world):
    spawn_ranks(_mappings, world, (), backend="gloo")


# ------------------------------------------------------------------------------------------------ sliced initialisation
def _sliced_init(rank, world, stride):
    mpu.initialize_model_parallel(world)
    out_features, in_features = 12 * world, 10 * world

    def same_everywhere(w):
        return torch.nn.init.normal_(w, generator=torch.Generator().manual_seed(99))

    full = same_everywhere(torch.empty(out_features, in_features))
    # rows (dimension 0): rank r keeps pieces r, r + world, ... of stride * world equal pieces
    per_part = out_features // world
    w = torch.empty(per_part, in_features)
    master = tp_layers._initialize_affine_weight(w, out_features, in_features, per_part, 0, same_everywhere, stride=stride, return_master_weight=True)
    assert torch.equal(master, full)
    piece = per_part // stride
    want = torch.cat([full[(rank + k * world) * piece:(rank + k * world + 1) * piece] for k in range(stride)], dim=0)
    assert torch.equal(w, want)
    # columns (dimension 1)
    per_part = in_features // world
    w = torch.empty(out_features, per_part)
    assert tp_layers._initialize_affine_weight(w, out_features, in_features, per_part, 1, same_everywhere, stride=stride) is None
    piece = per_part // stride
    want = torch.cat([full[:, (rank + k * world) * piece:(rank + k * world + 1) * piece] for k in range(stride)], dim=1)
    assert torch.equal(w, want)
    mpu.destroy_model_parallel()


@pytest.mark.parametrize("stride", [1, 2])
def test_each_rank_keeps_its_slices_of_the_common_draw(stride):
    spawn_ranks(_sliced_init, 2, (stride,), backend="gloo")


# ------------------------------------------------------------------------------------------------ layers against the dense formulas
def _linear_gradients(rank, world):
    mpu.initialize_model_parallel(world)
    batch, n_in, n_out = 7, 6 * world, 8 * world
    torch.manual_seed(12345)
    x = torch.randn(batch, n_in)
    dldy = torch.randn(batch, n_out)  # loss = sum(Y * dldy)

    torch.manual_seed(1)
    col = mpu.ColumnParallelLinear(n_in, n_out, keep_master_weight_for_test=True)
    xin = x.clone().requires_grad_()
    (col(xin) * dldy).sum().backward()
    a = col.master_weight
    # dL/dA = dL/dY^T X, dL/db = column sums of dL/dY, dL/dX = dL/dY A: this rank holds its rows of the first two
    rows = slice(rank * (n_out // world), (rank + 1) * (n_out // world))
    torch.testing.assert_close(col.weight.grad, (dldy.t() @ x)[rows], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(col.bias.grad, dldy.sum(0)[rows], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(xin.grad, dldy @ a, atol=1e-5, rtol=1e-5)
    # without the gather every rank keeps its own columns of Y
    torch.manual_seed(1)
    local = mpu.ColumnParallelLinear(n_in, n_out, gather_output=False, bias=False, keep_master_weight_for_test=True)
    assert local.bias is None
    torch.testing.assert_close(local(x), (x @ a.t())[:, rows], atol=1e-5, rtol=1e-5)

    torch.manual_seed(2)
    row = mpu.RowParallelLinear(n_in, n_out, keep_master_weight_for_test=True)
    xin = x.clone().requires_grad_()
    (row(xin) * dldy).sum().backward()
    a = row.master_weight
    cols = slice(rank * (n_in // world), (rank + 1) * (n_in // world))
    torch.testing.assert_close(row.weight.grad, (dldy.t() @ x)[:, cols], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(row.bias.grad, dldy.sum(0), atol=1e-5, rtol=1e-5)  # the bias is whole on every rank
    torch.testing.assert_close(xin.grad, dldy @ a, atol=1e-5, rtol=1e-5)
    # input already split: every rank feeds its own columns of X
    torch.manual_seed(2)
    pre_split = mpu.RowParallelLinear(n_in, n_out, input_is_parallel=True, bias=False, keep_master_weight_for_test=True)
    torch.testing.assert_close(pre_split(x[:, cols].contiguous()), x @ a.t(), atol=1e-5, rtol=1e-5)
    # the layers report the whole weight on request
    torch.testing.assert_close(row.get_master_weight(), a)
    torch.testing.assert_close(col.get_master_weight(), col.master_weight)
    with pytest.raises(AssertionError):
        mpu.ColumnParallelLinear(n_in, n_out + 1)  # features must divide among the ranks
    with pytest.raises(AssertionError):
        mpu.RowParallelLinear(n_in + 1, n_out)
    mpu.destroy_model_parallel()


def test_parallel_linear_gradients_follow_the_dense_formulas():
    spawn_ranks(_linear_gradients, 2, (), backend="gloo")


def _embeddings(rank, world):
    mpu.initialize_model_parallel(world)
    vocab, hidden, batch, seq = 6 * world, 4 * world, 3, 5
    torch.manual_seed(5)
    tokens = torch.randint(0, vocab, (batch, seq))
    weights = torch.randn(batch, seq, hidden)

    def draw(w):
        return torch.nn.init.normal_(w, generator=torch.Generator().manual_seed(7))

    dense = torch.nn.Embedding(vocab, hidden)
    draw(dense.weight.data)
    (dense(tokens) * weights).sum().backward()

    by_vocab = mpu.VocabParallelEmbedding(vocab, hidden, init_method=draw)
    out = by_vocab(tokens)
    torch.testing.assert_close(out, dense(tokens))
    (out * weights).sum().backward()
    rows = slice(rank * (vocab // world), (rank + 1) * (vocab // world))
    assert (by_vocab.vocab_start_index, by_vocab.vocab_end_index) == (rows.start, rows.stop)
    torch.testing.assert_close(by_vocab.weight.grad, dense.weight.grad[rows])

    by_width = mpu.ParallelEmbedding(vocab, hidden, init_method=draw)
    out = by_width(tokens)
    torch.testing.assert_close(out, dense(tokens))
    (out * weights).sum().backward()
    cols = slice(rank * (hidden // world), (rank + 1) * (hidden // world))
    torch.testing.assert_close(by_width.weight.grad, dense.weight.grad[:, cols])

    # a padding row gives what the dense layer gives and receives no gradient, whichever rank holds it
    pad = vocab - 1
    dense_pad = torch.nn.Embedding(vocab, hidden, padding_idx=pad)
    draw(dense_pad.weight.data)
    padded = mpu.VocabParallelEmbedding(vocab, hidden, padding_idx=pad, init_method=draw)
    with_pad = torch.cat([tokens, torch.full((batch, 1), pad)], dim=1)
    out = padded(with_pad)
    torch.testing.assert_close(out, dense_pad(with_pad))
    out.sum().backward()
    dense_pad(with_pad).sum().backward()
    torch.testing.assert_close(padded.weight.grad, dense_pad.weight.grad[rows])
    if rank == world - 1:
        assert float(padded.weight.grad[pad - rows.start].abs().sum()) == 0.0
    with pytest.raises(AssertionError):
        mpu.VocabParallelEmbedding(vocab + 1, hidden)
    with pytest.raises(AssertionError):
        mpu.ParallelEmbedding(vocab, hidden + 1)
    mpu.destroy_model_parallel()


def test_embeddings_forward_and_backward_match_the_dense_table():
    spawn_ranks(_embeddings, 2, (), backend="gloo")


# ------------------------------------------------------------------------------------------------ loss on shards
def _cross_entropy(rank, world, scale):
    mpu.initialize_model_parallel(world)
    batch, seq, vocab = 4, 3, 5 * world
    torch.manual_seed(1234)
    logits = torch.randn(batch, seq, vocab) * scale
    target = torch.randint(0, vocab, (batch, seq))
    dense = logits.clone().requires_grad_()
    want = F.cross_entropy(dense.view(-1, vocab), target.view(-1), reduction="none").view_as(target).mean()
    want.backward()
    shard = logits[..., rank * 5:(rank + 1) * 5].clone().requires_grad_()
    got = mpu.vocab_parallel_cross_entropy(shard, target).mean()
    got.backward()
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(shard.grad, dense.grad[..., rank * 5:(rank + 1) * 5], atol=1e-6, rtol=1e-5)
    assert torch.isfinite(got)
    mpu.destroy_model_parallel()


@pytest.mark.parametrize("scale", [1.0, 1000.0])
def test_loss_on_vocabulary_shards_equals_the_dense_loss(scale):
    spawn_ranks(_cross_entropy, 2, (scale,), backend="gloo")


# ------------------------------------------------------------------------------------------------ random streams
def _random_streams(rank, world):
    mpu.initialize_model_parallel(world)
    mpu.model_parallel_cuda_manual_seed(12345)
    tracker = mpu.get_cuda_rng_tracker()
    default_draw = torch.rand(3)
    with tracker.fork():
        parallel_draw = torch.rand(3)
    everyone_default = [torch.empty(3) for _ in range(world)]
    everyone_parallel = [torch.empty(3) for _ in range(world)]
    dist.all_gather(everyone_default, default_draw)
    dist.all_gather(everyone_parallel, parallel_draw)
    assert all(torch.equal(everyone_default[0], t) for t in everyone_default)   # e.g. dropout on replicated activations
    assert len({tuple(t.tolist()) for t in everyone_parallel}) == world         # e.g. dropout on sharded activations
    # seeding again restarts both streams
    mpu.model_parallel_cuda_manual_seed(12345)
    assert torch.equal(torch.rand(3), default_draw)
    with tracker.fork():
        assert torch.equal(torch.rand(3), parallel_draw)
    # the model-parallel stream is the generator seeded with seed + 2718 + rank
    torch.manual_seed(12345 + 2718 + rank)
    assert torch.equal(torch.rand(3), parallel_draw)

    # checkpoint replays both streams: gradients equal those of the same forward kept in memory
    lin = torch.nn.Linear(8, 8)

    def block(t):
        t = F.dropout(lin(t), 0.5, training=True)            # default stream
        with tracker.fork():
            return F.dropout(t, 0.5, training=True)          # model-parallel stream

    x = torch.randn(4, 8)
    mpu.model_parallel_cuda_manual_seed(7)
    a = x.clone().requires_grad_()
    block(a).sum().backward()
    kept, lin_grad = a.grad.clone(), lin.weight.grad.clone()
    lin.zero_grad()
    mpu.model_parallel_cuda_manual_seed(7)
    b = x.clone().requires_grad_()
    out = mpu.checkpoint(block, b)
    torch.rand(5)                       # whatever is drawn between forward and backward
    with tracker.fork():
        torch.rand(5)
    after_default, after_parallel = torch.get_rng_state(), tracker.get_states()
    out.sum().backward()
    assert torch.equal(b.grad, kept) and torch.equal(lin.weight.grad, lin_grad)
    # ... and leaves the streams where the program had them
    assert torch.equal(torch.get_rng_state(), after_default)
    name = next(iter(after_parallel))
    assert torch.equal(tracker.get_states()[name], after_parallel[name])
    mpu.destroy_model_parallel()


def test_two_random_streams_and_the_checkpoint_that_replays_them():
    spawn_ranks(_random_streams, 2, (), backend="gloo")


def _checkpoint_under_autocast(rank, world):
    mpu.initialize_model_parallel(world)
    mpu.model_parallel_cuda_manual_seed(1)
    lin1, lin2 = torch.nn.Linear(8, 8), torch.nn.Linear(8, 8)

    def block(t):
        return lin2(torch.tanh(lin1(t)))

    x = torch.randn(4, 8)
    a, b = x.clone().requires_grad_(), x.clone().requires_grad_()
    with torch.autocast("cpu", dtype=torch.bfloat16):
        kept = block(a)
        replayed = mpu.checkpoint(block, b)
    assert replayed.dtype == torch.bfloat16
    kept.float().sum().backward()
    grads = [p.grad.clone() for p in (*lin1.parameters(), *lin2.parameters())]
    for p in (*lin1.parameters(), *lin2.parameters()):
        p.grad = None
    replayed.float().sum().backward()  # the repetition runs with autocast on again
    for p, g in zip((*lin1.parameters(), *lin2.parameters()), grads):
        torch.testing.assert_close(p.grad, g, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(b.grad, a.grad, atol=1e-6, rtol=1e-5)
    mpu.destroy_model_parallel()


def test_checkpoint_replays_under_the_forwards_autocast_state():
    spawn_ranks(_checkpoint_under_autocast, 1, (), backend="gloo")
