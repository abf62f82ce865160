"""Token streams for the LM benchmarks.  Only the synthetic stream is available offline: a fixed random sequence of
2,049,990 token ids in [1, 10000) (the size of wikitext-2's training split), cut into ``[batch, seq_len]`` windows."""

from collections import namedtuple

import torch
from torch.utils.data import DataLoader

DatasetsInfo = namedtuple("DatasetsInfo", ["ntokens", "train_dataset", "valid_dataset", "test_dataset"])


def get_synthetic_datasets(vocab: int = 10000, n: int = 2049990, seed: int = 0) -> DatasetsInfo:
    g = torch.Generator().manual_seed(seed)
    data = torch.randint(1, vocab, (n,), generator=g)
    return DatasetsInfo(vocab, data, data[: n // 10], data[: n // 10])


def get_real_datasets() -> DatasetsInfo:
    raise RuntimeError("wikitext-2 is not bundled and there is no network access; use --use_synthetic_data")


def get_dataloaders(info: DatasetsInfo, batch_size: int, seq_len: int, rank: int = 0, world: int = 1, max_batches: int = 0):
    """Batches of ``{"input": [B, S], "target": [B, S]}``; ranks read disjoint strides of the stream."""

    def make(data):
        per = batch_size * (seq_len + 1)
        n = data.numel() // per
        if max_batches:
            n = min(n, max_batches * world)
        windows = data[: n * per].view(n, batch_size, seq_len + 1)[rank::world]
        return DataLoader([{"input": w[:, :-1].contiguous(), "target": w[:, 1:].contiguous()} for w in windows], batch_size=None)

    return make(info.train_dataset), make(info.valid_dataset), make(info.test_dataset)
