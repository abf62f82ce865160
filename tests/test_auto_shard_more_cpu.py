"""shard_model on models that are not sequential (cases of the reference's tests/experimental/nn/test_auto_shard.py): sub-modules
with data-dependent control flow, which symbolic tracing cannot enter, are kept whole as leaves and the shards still compose
to the model; a transformer language model with a mask as second input runs shard by shard."""
import math

import pytest
import torch
from torch import nn

from fairscale_b200.experimental.nn.auto_shard import shard_model


class _Branch(nn.Module):
    def __init__(self, features):
        super().__init__()
        self.left, self.right = nn.Linear(features, features), nn.Linear(features, features)

    def forward(self, x):
        return self.left(x) if x.sum() > 1000 else self.right(x)  # depends on the data


class _Branched(nn.Module):
    def __init__(self, features):
        super().__init__()
        torch.manual_seed(0)
        self.net = nn.ModuleList([_Branch(features) for _ in range(10)])

    def forward(self, x):
        for module in self.net:
            x = module(x)
        return x


@pytest.mark.parametrize("shards", [2, 3, 5])
def test_data_dependent_branches_are_kept_whole(shards):
    model = _Branched(10)
    pieces = shard_model(model, shards)
    assert len(pieces) == shards
    for x in (torch.randn(3, 10), torch.full((3, 10), 100.0)):  # both sides of the condition
        out = x
        for piece in pieces:
            out = piece(out)
        torch.testing.assert_close(out, model(x))
    # every parameter landed in exactly one shard
    assert sum(p.numel() for piece in pieces for p in piece.parameters()) == sum(p.numel() for p in model.parameters())
    sizes = [sum(p.numel() for p in piece.parameters()) for piece in pieces]
    assert max(sizes) <= 2 * (sum(sizes) / shards) + 220  # roughly balanced; a branch (220 parameters) is never split


class _Positional(nn.Module):
    def __init__(self, d_model, max_len=64):
        super().__init__()
        pe = torch.zeros(max_len, d_model)
        position = torch.arange(0, max_len, dtype=torch.float).unsqueeze(1)
        div = torch.exp(torch.arange(0, d_model, 2).float() * (-math.log(10000.0) / d_model))
        pe[:, 0::2], pe[:, 1::2] = torch.sin(position * div), torch.cos(position * div)
        self.register_buffer("pe", pe.unsqueeze(1))

    def forward(self, x):
        return x + self.pe[: x.size(0)]


class _LM(nn.Module):
    def __init__(self, ntoken=301, ninp=16, nhead=2, nhid=16, nlayers=1):
        super().__init__()
        torch.manual_seed(0)
        self.pos_encoder = _Positional(ninp)
        self.transformer_encoder = nn.TransformerEncoder(nn.TransformerEncoderLayer(ninp, nhead, nhid, 0.0), nlayers)
        self.encoder = nn.Embedding(ntoken, ninp)
        self.ninp = ninp
        self.decoder = nn.Linear(ninp, ntoken)

    def forward(self, *args):
        src, mask = args[0], args[1]
        src = self.pos_encoder(self.encoder(src) * math.sqrt(self.ninp))
        return self.decoder(self.transformer_encoder(src, mask))


def test_language_model_with_two_inputs_runs_shard_by_shard():
    model = _LM().eval()
    pieces = shard_model(model)
    assert len(pieces) == 2
    assert sum(p.numel() for piece in pieces for p in piece.parameters()) == sum(p.numel() for p in model.parameters())
    src = torch.randint(1, 301, (12, 4))
    mask = torch.triu(torch.full((12, 12), float("-inf")), diagonal=1)
    value = [src, mask]
    for piece in pieces:
        value = piece(*value) if isinstance(value, (list, tuple)) else piece(value)
    assert value.shape == (12, 4, 301)
    with torch.no_grad():
        torch.testing.assert_close(value, model(src, mask), atol=1e-5, rtol=1e-4)
