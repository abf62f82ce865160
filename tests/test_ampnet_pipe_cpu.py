"""AMPnetPipe on gloo ranks: with one batch in flight per stage boundary the loss falls; 1-stage run equals plain SGD."""
import torch
import torch.distributed as dist
from torch import nn
from torch.utils.data import DataLoader, Dataset

from fairscale_b200.experimental.nn.ampnet_pipe import AMPnetPipe
from fairscale_b200.fair_dev.testing.testing import spawn_ranks


class _Data(Dataset):
    def __init__(self, n=24):
        g = torch.Generator().manual_seed(0)
        self.x = torch.randn(n, 4, 8, generator=g)
        w = torch.randn(8, 3, generator=g)
        self.y = (self.x @ w).argmax(-1)

    def __len__(self):
        return len(self.x)

    def __getitem__(self, i):
        return {"input": self.x[i], "target": self.y[i]}


class _Delegate:
    def __init__(self):
        self.losses, self.saved = [], 0

    def transform_input(self, b):
        return b["input"].squeeze(0)

    def transform_target(self, b):
        return b["target"].squeeze(0)

    def transform_output_before_loss(self, out):
        return out

    def log_loss(self, batch, loss, count):
        self.losses.append(float(loss.detach()))

    def check_and_save_weights(self, n):
        self.saved += 1


def _layers():
    torch.manual_seed(1)
    return nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 3))


def _worker(rank, world, balance):
    pipe = AMPnetPipe(_layers(), balance=balance, chunks=1, checkpoint="never")
    opt = torch.optim.SGD(pipe.partition.parameters(), lr=0.2) if pipe.partition is not None else None
    delegate = _Delegate()
    for _ in range(3):
        pipe.interleave(DataLoader(_Data(), batch_size=1), nn.CrossEntropyLoss(), opt, delegate, min_update_interval=1)
    if rank == len(balance) - 1:
        first, lastl = sum(delegate.losses[:12]) / 12, sum(delegate.losses[-12:]) / 12
        assert lastl < 0.7 * first, (first, lastl)
        assert delegate.saved == 72
        if len(balance) == 1:  # no staleness with one stage: identical to a plain training loop
            ref = _layers()
            ropt = torch.optim.SGD(ref.parameters(), lr=0.2)
            losses = []
            for _ in range(3):
                for b in DataLoader(_Data(), batch_size=1):
                    loss = nn.CrossEntropyLoss()(ref(b["input"].squeeze(0)), b["target"].squeeze(0))
                    ropt.zero_grad(); loss.backward(); ropt.step()
                    losses.append(float(loss))
            torch.testing.assert_close(torch.tensor(losses), torch.tensor(delegate.losses))
    dist.barrier()


def test_ampnet_three_stages_trains():
    spawn_ranks(_worker, 3, ([2, 2, 1],), backend="gloo")


def test_ampnet_single_stage_equals_sgd():
    spawn_ranks(_worker, 2, ([5],), backend="gloo")
