"""OSS + ShardedDataParallel on 2 gloo ranks must reproduce torch DDP's per-step loss to 1e-5
(fp32, 2-layer d256 decoder LM, seq 64, batch 8 per rank, Adam lr 1e-3, 20 steps)."""
import copy

import pytest
import torch
import torch.distributed as dist

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.nn.data_parallel import ShardedDataParallel
from fairscale_b200.optim import OSS

from _models import TinyDecoderLM, lm_loss


def _run(rank, world_size, steps, buffer_size):
    torch.manual_seed(0)
    torch.set_num_threads(2)
    base = TinyDecoderLM()
    ddp_model = torch.nn.parallel.DistributedDataParallel(copy.deepcopy(base))
    ddp_opt = torch.optim.Adam(ddp_model.parameters(), lr=1e-3)

    sdp_base = copy.deepcopy(base)
    oss = OSS(sdp_base.parameters(), optim=torch.optim.Adam, lr=1e-3)
    sdp_model = ShardedDataParallel(sdp_base, oss, reduce_buffer_size=buffer_size)

    gen = torch.Generator().manual_seed(0)
    data = torch.randint(0, 10000, (steps, world_size, 8, 64), generator=gen)
    for step in range(steps):
        tokens = data[step, rank]
        ddp_opt.zero_grad()
        l_ref = lm_loss(ddp_model(tokens), tokens)
        l_ref.backward()
        ddp_opt.step()

        sdp_model.zero_grad()
        l_new = lm_loss(sdp_model(tokens), tokens)
        l_new.backward()
        oss.step()
        assert abs(l_ref.item() - l_new.item()) <= 1e-5, (step, l_ref.item(), l_new.item())
    for a, b in zip(ddp_model.module.parameters(), sdp_base.parameters()):
        torch.testing.assert_close(a, b, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("buffer_size", [0, 2**23])
def test_oss_sdp_matches_ddp_20_steps(buffer_size):
    spawn_ranks(_run, 2, (20, buffer_size), backend="gloo", timeout=600)
