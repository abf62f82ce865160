"""MoE language model on 2 gloo ranks: trains, and expert gradients stay rank-local while dense ones can be averaged."""
import torch
import torch.distributed as dist

from fairscale_b200.fair_dev.testing.testing import spawn_ranks


def _worker(rank, world):
    from fairscale_b200.models.moe_lm import MoELM, MoELMConfig

    torch.manual_seed(0)
    cfg = MoELMConfig(vocab_size=128, d_model=32, n_heads=2, n_layers=4, ffn=64, max_seq=16, num_local_experts=2)
    model = MoELM(cfg)
    assert sum(1 for b in model.blocks if hasattr(b, "moe")) == 2
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)
    g = torch.Generator().manual_seed(10 + rank)
    toks = torch.randint(0, 128, (4, 17), generator=g)
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = model(x, y)
        loss.backward()
        for p in model.dense_parameters():
            dist.all_reduce(p.grad)
            p.grad /= world
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]
    assert all(p.grad is not None for p in model.expert_parameters())


def test_moe_lm_trains_on_two_ranks():
    spawn_ranks(_worker, 2, (), backend="gloo")
