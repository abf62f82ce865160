"""Tensor-parallel Llama on 2 gloo ranks: loss and a step of SGD equal the single-rank model under the same seed."""
import torch
import torch.distributed as dist

from fairscale_b200.fair_dev.testing.testing import spawn_ranks


def _run(rank, world, tp):
    from fairscale_b200.models.tp_llama import TPLlama, TPLlamaConfig
    from fairscale_b200.nn.model_parallel import destroy_model_parallel, initialize_model_parallel

    initialize_model_parallel(tp)
    torch.manual_seed(1234)
    cfg = TPLlamaConfig.tiny()
    model = TPLlama(cfg)
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, cfg.vocab_size, (2, 9), generator=g)
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    losses = []
    for _ in range(3):
        opt.zero_grad()
        loss = model(x, y)
        loss.backward()
        if tp > 1:  # replicated parameters (norm weights) see different token shards: sum their gradients
            for n, p in model.named_parameters():
                if "norm" in n and p.grad is not None:
                    dist.all_reduce(p.grad)
        opt.step()
        losses.append(float(loss.detach()))
    destroy_model_parallel()
    return losses


def _worker(rank, world):
    multi = _run(rank, world, 2)
    # the same model with model-parallel size 1: every rank holds everything, no communication inside the layers
    single = _run(rank, world, 1)
    torch.testing.assert_close(torch.tensor(multi), torch.tensor(single), rtol=1e-4, atol=1e-5)
    assert multi[-1] < multi[0]


def test_tp_llama_matches_single_rank():
    spawn_ranks(_worker, 2, (), backend="gloo")
