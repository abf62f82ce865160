"""Synthetic fixed-length token dataset used by the asynchronous-pipeline benchmark (reference:
benchmarks/experimental/benchmark_dataset.py:10-66)."""

import torch
from torch.utils.data import Dataset


def collate_sentences_lm(samples):
    if len(samples) == 0:
        return {}
    src = torch.stack([s["source"] for s in samples])
    tgt = torch.stack([s["target"] for s in samples])
    return {"id": torch.tensor([s["id"] for s in samples]), "input": src, "target": tgt, "ntokens": int(tgt.numel())}


class BenchmarkLMDataset(Dataset):
    """``total_samples`` random sequences of ``max_source_positions`` tokens; the target is the input shifted by one."""

    def __init__(self, vocab_size: int = 10000, max_source_positions: int = 1024, total_samples: int = 10000, seed: int = 0):
        self.vocab_size, self.max_source_positions, self.total_samples = vocab_size, max_source_positions, total_samples
        g = torch.Generator().manual_seed(seed)
        self.data = torch.randint(1, vocab_size, (total_samples, max_source_positions + 1), generator=g)

    def __getitem__(self, index):
        row = self.data[index]
        return {"id": index, "source": row[:-1], "target": row[1:]}

    def __len__(self):
        return self.total_samples
