"""FSDP around modules whose outputs are not plain tensors (cases of the reference's
tests/nn/data_parallel/test_fsdp_hf_transformer_eval.py and test_fsdp_input.py, on gloo ranks): an inner wrapped
``nn.Transformer`` that returns a dataclass-style ordered mapping indexed by position, auto-wrapped by a policy that picks the
transformer only; and a randomly initialised GPT-2 from the ``transformers`` library (if importable) wrapped block by block,
evaluated and trained for a step against the unwrapped copy."""
from collections import OrderedDict
from dataclasses import dataclass
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn import FullyShardedDataParallel as FSDP
from fairscale_b200.nn import auto_wrap, enable_wrap

CPU = dict(compute_device=torch.device("cpu"))


class ModelOutput(OrderedDict):
    """Ordered mapping that also answers integer indices, filled from its dataclass fields (the convention of model outputs
    in the transformers library)."""

    def to_tuple(self):
        return tuple(self[k] for k in self.keys())

    def __post_init__(self):
        for field in getattr(self, "__dataclass_fields__"):
            value = getattr(self, field)
            if value is not None:
                self[field] = value

    def __getitem__(self, k):
        return dict(self.items())[k] if isinstance(k, str) else self.to_tuple()[k]


@dataclass
class TransformerOutput(ModelOutput):
    output: torch.FloatTensor = None


class TransformerWithCustomOutput(nn.Transformer):
    def forward(self, *args, **kwargs):
        return TransformerOutput(output=super().forward(*args, **kwargs))


class TransformerWithLMHead(nn.Module):
    def __init__(self, d_vocab=50, d_model=16):
        super().__init__()
        torch.manual_seed(0)
        self.d_vocab = d_vocab
        self.embed_tokens = nn.Embedding(d_vocab, d_model)
        self.transformer = TransformerWithCustomOutput(d_model, nhead=2, num_encoder_layers=2, num_decoder_layers=2, dim_feedforward=32, dropout=0.0)
        self.output_proj = nn.Linear(d_model, d_vocab)

    def forward(self, source_seq, target_seq):
        output = self.transformer(self.embed_tokens(source_seq), self.embed_tokens(target_seq))
        return self.output_proj(output[0])  # an integer key, as user code of such models writes it


def _wrap_transformer_only(module, recurse, **kwargs):
    return True if recurse else isinstance(module, nn.Transformer)


def _custom_output(rank, world):
    plain = TransformerWithLMHead()
    model = copy.deepcopy(plain)
    with enable_wrap(wrapper_cls=FSDP, auto_wrap_policy=_wrap_transformer_only, **CPU):
        model = auto_wrap(model)
    model = FSDP(model, **CPU)
    assert isinstance(model.transformer, FSDP) and not isinstance(model.embed_tokens, FSDP)
    g = torch.Generator().manual_seed(rank)
    src, tgt = torch.randint(50, (7, 2), generator=g), torch.randint(50, (7, 2), generator=g)
    model.eval()
    plain.eval()
    with torch.no_grad():
        torch.testing.assert_close(model(src, tgt), plain(src, tgt), atol=1e-5, rtol=1e-4)
    # and it trains: the pre-backward hooks found the tensor inside the mapping
    model.train()
    model(src, tgt).logsumexp(-1).mean().backward()
    assert all(p.grad is not None for p in model.parameters())


@pytest.mark.parametrize("world", [1, 2])
def test_inner_unit_returning_an_ordered_mapping(world):
    spawn_ranks(_custom_output, world, (), backend="gloo")


def _gpt2(rank, world):
    transformers = pytest.importorskip("transformers")
    config = transformers.GPT2Config(vocab_size=64, n_positions=16, n_embd=16, n_layer=2, n_head=2, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    torch.manual_seed(0)
    plain = transformers.GPT2LMHeadModel(config)
    model = copy.deepcopy(plain)
    for i, block in enumerate(model.transformer.h):
        model.transformer.h[i] = FSDP(block, **CPU)
    model = FSDP(model, **CPU)
    tokens = torch.randint(64, (2, 12), generator=torch.Generator().manual_seed(rank))
    model.eval()
    plain.eval()
    with torch.no_grad():
        torch.testing.assert_close(model(tokens).logits, plain(tokens).logits, atol=1e-5, rtol=1e-4)
    # one training step against DistributedDataParallel on the unwrapped copy (the output embedding is tied to the input one)
    model.train()
    plain.train()
    ddp = nn.parallel.DistributedDataParallel(plain)
    opts = [torch.optim.SGD(m.parameters(), lr=0.1) for m in (model, ddp)]
    losses = []
    for m, opt in zip((model, ddp), opts):
        out = m(tokens, labels=tokens)
        out.loss.backward()
        opt.step()
        losses.append(float(out.loss))
    assert abs(losses[0] - losses[1]) < 1e-5
    full = model.state_dict()
    for k, v in plain.state_dict().items():
        torch.testing.assert_close(full[k], v, atol=1e-5, rtol=1e-4)
    dist.barrier()


def test_gpt2_from_the_transformers_library_block_by_block():
    pytest.importorskip("transformers")
    spawn_ranks(_gpt2, 2, (), backend="gloo")
