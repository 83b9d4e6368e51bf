"""Synthetic token source (``dataset_impl: synthetic``): uniform random ids in [0, vocab) from a
seed, ``seq_length + 1`` tokens per sample so that labels are the inputs shifted by one.  Sample
``i`` depends only on ``(seed, i)``: every rank and every restart sees the same stream."""
from __future__ import annotations

import numpy as np
import torch


class SyntheticDataset(torch.utils.data.Dataset):
    def __init__(self, num_samples: int, seq_length: int, vocab_size: int, seed: int = 1234):
        self.num_samples, self.seq_length, self.vocab_size, self.seed = num_samples, seq_length, vocab_size, seed

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx):
        rng = np.random.Generator(np.random.Philox(key=self.seed, counter=[0, 0, 0, int(idx)]))
        return {"text": rng.integers(0, self.vocab_size, size=self.seq_length + 1, dtype=np.int64)}
