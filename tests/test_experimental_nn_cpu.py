"""experimental.nn on CPU: MEVO vs un-tiled oracle, OffloadModel vs the plain model, auto_shard, SyncBatchNorm."""
import copy

import pytest
import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from fairscale_b200.experimental.nn import BaselineSoftmaxNllLoss, MemoryEfficientVocabOutput, OffloadModel, SyncBatchNorm
from fairscale_b200.experimental.nn.auto_shard import shard_model
from fairscale_b200.experimental.optim import DynamicLossScaler
from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.checkpoint import checkpoint_wrapper


@pytest.mark.parametrize("scale", [None, 16.0])
@pytest.mark.parametrize("reduction", ["sum", "mean"])
def test_mevo_matches_baseline(scale, reduction):
    torch.manual_seed(0)
    tokens, d, vocab = 48, 16, 200  # not multiples of the tile sizes
    w = nn.Parameter(torch.randn(vocab, d) * 0.3)
    x = torch.randn(tokens, d, requires_grad=True)
    t = torch.randint(0, vocab, (tokens,))
    mevo = MemoryEfficientVocabOutput(w, tile_factor=4, reduction=reduction, scale=scale)
    loss = mevo(x, t)
    loss.backward()
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    ref = BaselineSoftmaxNllLoss(w, scale=scale)(x, t)
    if reduction == "mean":
        ref = ref / tokens
    ref.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(gx, x.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gw, w.grad, rtol=1e-4, atol=1e-5)
    assert mevo.trigger.trigger.grad is not None and float(mevo.trigger.trigger.grad) == 0.0
    mevo.eval()
    assert mevo(x, None).shape == (tokens, vocab)


def _mlp():
    torch.manual_seed(3)
    return nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 16), nn.BatchNorm1d(16), nn.ReLU(), nn.Linear(16, 4))


@pytest.mark.parametrize("ckpt,mb", [(False, 1), (True, 1), (True, 2)])
def test_offload_model_matches_plain(ckpt, mb):
    ref = _mlp()
    if mb > 1:  # batch statistics differ per micro-batch
        ref[3] = nn.Identity()
    model = copy.deepcopy(ref)
    off = OffloadModel(model, torch.device("cpu"), torch.device("cpu"), num_slices=3, checkpoint_activation=ckpt, num_microbatches=mb)
    assert len(off.model_slices) == 3
    opt_ref = torch.optim.SGD(ref.parameters(), lr=0.1)
    opt = torch.optim.SGD(off.parameters(), lr=0.1)
    for step in range(3):
        torch.manual_seed(step)
        x = torch.randn(6, 8, requires_grad=True)
        x2 = x.detach().clone().requires_grad_()
        if mb > 1:
            want = torch.cat([ref(c) for c in x2.chunk(mb)])
        else:
            want = ref(x2)
        got = off(x)
        torch.testing.assert_close(got, want)
        want.pow(2).sum().backward()
        got.pow(2).sum().backward()
        off.sync()
        torch.testing.assert_close(x.grad, x2.grad)
        for a, b in zip(off.parameters(), ref.parameters()):
            torch.testing.assert_close(a.grad, b.grad, rtol=1e-5, atol=1e-6)
        opt.step(); opt_ref.step(); opt.zero_grad(); opt_ref.zero_grad()
    for a, b in zip(off.state_dict().values(), ref.state_dict().values()):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    with pytest.raises(RuntimeError):
        OffloadModel(_mlp(), torch.device("cpu"), num_microbatches=2)
    with pytest.raises(TypeError):
        OffloadModel(nn.Linear(2, 2), torch.device("cpu"))


class _Res(nn.Module):
    def __init__(self):
        super().__init__()
        self.a, self.b, self.c, self.d = nn.Linear(8, 8), nn.Linear(8, 8), nn.Linear(8, 8), nn.Linear(8, 2)

    def forward(self, x):
        h = self.a(x)
        h = h + self.b(torch.relu(h))  # a cut inside this residual is illegal
        h = torch.relu(self.c(h))
        return self.d(h)


def test_auto_shard_composes_to_the_model():
    torch.manual_seed(0)
    model = _Res()
    shards = shard_model(model, 3)
    assert 2 <= len(shards) <= 3
    x = torch.randn(5, 8)
    y = x
    for s in shards:
        y = s(y)
    torch.testing.assert_close(y, model(x))
    assert sum(p.numel() for s in shards for p in s.parameters()) == sum(p.numel() for p in model.parameters())
    seq = nn.Sequential(*[nn.Linear(4, 4) for _ in range(6)])
    shards = shard_model(seq, 3)
    assert len(shards) == 3 and [sum(p.numel() for p in s.parameters()) for s in shards] == [40, 40, 40]


def _syncbn_rank(rank, world, wrap):
    torch.manual_seed(0)
    full = torch.randn(8, 3, 4, 4)
    ref_bn = nn.BatchNorm2d(3)
    ref_in = full.clone().requires_grad_()
    ref_out = ref_bn(ref_in)
    (ref_out * torch.arange(8.0).view(8, 1, 1, 1)).sum().backward()
    bn = SyncBatchNorm.convert_sync_batchnorm(nn.Sequential(nn.BatchNorm2d(3)))
    assert isinstance(bn[0], SyncBatchNorm)
    mod = checkpoint_wrapper(bn) if wrap else bn
    x = full[rank * 4 : rank * 4 + 4].clone().requires_grad_()
    out = mod(x)
    (out * torch.arange(8.0)[rank * 4 : rank * 4 + 4].view(4, 1, 1, 1)).sum().backward()
    torch.testing.assert_close(out, ref_out[rank * 4 : rank * 4 + 4], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(x.grad, ref_in.grad[rank * 4 : rank * 4 + 4], rtol=1e-4, atol=1e-5)
    g = bn[0].weight.grad.clone()
    dist.all_reduce(g)
    torch.testing.assert_close(g, ref_bn.weight.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(bn[0].running_mean, ref_bn.running_mean, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(bn[0].running_var, ref_bn.running_var, rtol=1e-4, atol=1e-6)
    assert int(bn[0].num_batches_tracked) == 1


@pytest.mark.parametrize("wrap", [False, True])
def test_sync_batchnorm_matches_full_batch(wrap):
    spawn_ranks(_syncbn_rank, 2, (wrap,), backend="gloo")


def test_dynamic_loss_scaler():
    model = nn.Linear(4, 2)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    scaler = DynamicLossScaler(init_scale=8.0, scale_window=2)
    scaler.scale(model(torch.ones(1, 4)).sum()).backward()
    g = model.weight.grad.clone()
    before = model.weight.detach().clone()
    scaler.step(opt)
    scaler.update()
    torch.testing.assert_close(model.weight, before - 0.1 * g / 8.0)
    opt.zero_grad()
    scaler.scale(model(torch.ones(1, 4)).sum()).backward()
    model.weight.grad[0, 0] = float("inf")
    before = model.weight.detach().clone()
    assert scaler.step(opt) is None and torch.equal(before, model.weight)
    assert scaler.loss_scale == 4.0
    tiny = DynamicLossScaler(init_scale=2e-4, min_loss_scale=1e-4)
    with pytest.raises(FloatingPointError):
        tiny.step(opt)
    assert scaler.state_dict() == {"loss_scale": 4.0}


@pytest.mark.parametrize("scale", [None, 8.0])
def test_mevo_three_pass_functions_compose_to_the_fused_loss(scale):
    """GetMax / GetSum / TargetScore (the reference's three passes) give the same loss and gradients as the single pass."""
    from fairscale_b200.experimental.nn.mevo import GetMaxFunction, GetSumFunction, MemoryEfficientVocabOutput, TargetScoreFunction

    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(40, 8))
    k = MemoryEfficientVocabOutput(w, tile_factor=2, scale=scale)
    x = torch.randn(6, 8, requires_grad=True)
    t = torch.randint(0, 40, (6,))
    mx = GetMaxFunction.apply(x, w, t, k)
    sm = GetSumFunction.apply(x, w, t, mx, k)
    loss = -((TargetScoreFunction.apply(x, w, t, k) - mx) - sm.log()).sum()
    ref = k(x, t)
    torch.testing.assert_close(loss, ref, atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(k.get_target_nlprob(x, w, t, mx, sm), ref, atol=1e-3, rtol=1e-4)
    gx, gw = torch.autograd.grad(loss, (x, w))
    rx, rw = torch.autograd.grad(ref, (x, w))
    torch.testing.assert_close(gx, rx, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(gw, rw, atol=1e-4, rtol=1e-4)


def test_auto_shard_transformer_reference_split():
    """A torch TransformerEncoder language model cut in two by parameter count: the reference records 5 998 600 and
    5 785 383 parameters for the two shards (tests/experimental/nn/test_auto_shard.py:82-99)."""
    import math

    class PositionalEncoding(nn.Module):
        def __init__(self, d_model, dropout=0.1, max_len=5000):
            super().__init__()
            self.dropout = nn.Dropout(p=dropout)
            pe = torch.zeros(max_len, d_model)
            position = torch.arange(0, max_len, dtype=torch.float).unsqueeze(1)
            div = torch.exp(torch.arange(0, d_model, 2).float() * (-math.log(10000.0) / d_model))
            pe[:, 0::2], pe[:, 1::2] = torch.sin(position * div), torch.cos(position * div)
            self.register_buffer("pe", pe.unsqueeze(0).transpose(0, 1))

        def forward(self, x):
            return self.dropout(x + self.pe[: x.size(0)])

    class TransformerModel(nn.Module):
        def __init__(self, ntoken, ninp, nhead, nhid, nlayers, dropout):
            super().__init__()
            self.pos_encoder = PositionalEncoding(ninp, dropout)
            self.transformer_encoder = nn.TransformerEncoder(nn.TransformerEncoderLayer(ninp, nhead, nhid, dropout), nlayers)
            self.encoder = nn.Embedding(ntoken, ninp)
            self.ninp = ninp
            self.decoder = nn.Linear(ninp, ntoken)

        def forward(self, *args):
            src = self.pos_encoder(self.encoder(args[0]) * math.sqrt(self.ninp))
            return self.decoder(self.transformer_encoder(src, args[1]))

    shards = shard_model(TransformerModel(28783, 200, 2, 200, 1, 0.2))
    assert len(shards) == 2
    assert [sum(p.numel() for p in s.parameters()) for s in shards] == [5998600, 5785383]


def test_dynamic_loss_scaler_schedule_window_tolerance_and_floor():
    model = nn.Linear(2, 1)
    opt = torch.optim.SGD(model.parameters(), lr=0.0)

    def run(scaler, overflow):
        opt.zero_grad()
        scaler.scale(model(torch.ones(1, 2)).sum()).backward()
        if overflow:
            model.weight.grad[0, 0] = float("nan")
        stepped = scaler.step(opt) is not None or not overflow
        if not overflow:
            scaler.update()
        return stepped

    # grows every `scale_window` clean steps
    s = DynamicLossScaler(init_scale=4.0, scale_window=3)
    scales = []
    for _ in range(7):
        run(s, False)
        scales.append(s.loss_scale)
    assert scales == [4.0, 4.0, 8.0, 8.0, 8.0, 16.0, 16.0], scales
    # with a tolerance, single overflows among many clean steps do not lower the scale; a burst does
    s = DynamicLossScaler(init_scale=64.0, scale_window=1000, tolerance=0.5)
    for _ in range(4):
        run(s, False)
    run(s, True)
    assert s.loss_scale == 64.0  # one overflow in five steps since the last change: below one half
    s2 = DynamicLossScaler(init_scale=64.0, scale_window=1000, tolerance=0.5)
    run(s2, False)
    run(s2, True)
    assert s2.loss_scale == 32.0  # one in two
    # the threshold is a floor for decreases; lists and tuples are scaled element-wise; state round trip
    s = DynamicLossScaler(init_scale=4.0, threshold=3.0)
    run(s, True)
    assert s.loss_scale == 3.0
    a, b = s.scale([torch.ones(1), torch.ones(1) * 2])
    assert float(a) == 3.0 and float(b) == 6.0 and isinstance(s.scale((torch.ones(1),)), tuple)
    other = DynamicLossScaler()
    other.load_state_dict(s.state_dict())
    assert other.loss_scale == 3.0
    # misuse is reported
    run(s, False)
    opt.zero_grad()
    s.scale(model(torch.ones(1, 2)).sum()).backward()
    s.unscale_(opt)
    with pytest.raises(RuntimeError):
        s.unscale_(opt)
    s.step(opt)
    with pytest.raises(RuntimeError):
        s.step(opt)
    with pytest.raises(RuntimeError):
        s.unscale_(opt)
    with pytest.raises(RuntimeError):
        DynamicLossScaler().step(opt, closure=lambda: 0)
