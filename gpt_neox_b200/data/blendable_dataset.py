"""Weighted interleave of several datasets (megatron/data/blendable_dataset.py:29-82): sample ``i``
comes from the dataset that is furthest below its target share so far (C++
``build_blending_indices``)."""
from __future__ import annotations

import time

import numpy as np
import torch

from ..utils.common import print_rank_0
from . import helpers


class BlendableDataset(torch.utils.data.Dataset):
    def __init__(self, datasets, weights):
        self.datasets = datasets
        num_datasets = len(datasets)
        assert num_datasets == len(weights)
        self.size = sum(len(d) for d in self.datasets)
        weights = np.array(weights, dtype=np.float64)
        assert weights.sum() > 0.0
        weights /= weights.sum()
        start_time = time.time()
        assert num_datasets < 255
        self.dataset_index = np.zeros(self.size, dtype=np.uint8)
        self.dataset_sample_index = np.zeros(self.size, dtype=np.int64)
        verbose = (not torch.distributed.is_initialized()) or torch.distributed.get_rank() == 0
        helpers.build_blending_indices(self.dataset_index, self.dataset_sample_index, weights, num_datasets,
                                       self.size, verbose)
        print_rank_0("> elapsed time for building blendable dataset indices: {:.2f} (sec)".format(
            time.time() - start_time))

    def __len__(self):
        return self.size

    def __getitem__(self, idx):
        try:
            dataset_idx = self.dataset_index[idx]
            sample_idx = self.dataset_sample_index[idx]
            return self.datasets[dataset_idx][sample_idx]
        except IndexError:
            new_idx = idx % len(self)
            print(f"WARNING: Got index out of bounds error with index {idx} - taking modulo of index instead "
                  f"({new_idx})")
            return self[new_idx]
