"""Weighted mixture of datasets.

Sample ``i`` of the mixture is drawn from the component that is, after ``i`` draws, furthest below its target
share (a deterministic low-discrepancy interleave, computed once for all ``sum(len(d))`` samples by the native
``build_blending_indices`` of csrc/data_helpers.cpp).  Two arrays describe the result: which component serves
sample ``i`` and which of its items.  Counterpart of megatron/data/blendable_dataset.py.
"""
from __future__ import annotations

import time

import numpy as np
import torch

from ..utils.common import print_rank_0
from . import helpers

_MAX_COMPONENTS = 254          # component ids are stored as uint8


class BlendableDataset(torch.utils.data.Dataset):
    def __init__(self, datasets, weights):
        if len(datasets) != len(weights):
            raise ValueError(f"{len(datasets)} datasets but {len(weights)} weights")
        if len(datasets) > _MAX_COMPONENTS:
            raise ValueError(f"at most {_MAX_COMPONENTS} datasets can be blended")
        share = np.asarray(weights, dtype=np.float64)
        if not share.sum() > 0.0:
            raise ValueError("blend weights must have a positive sum")
        share = share / share.sum()
        self.datasets = datasets
        self.size = int(sum(len(d) for d in datasets))
        self.dataset_index = np.zeros(self.size, dtype=np.uint8)
        self.dataset_sample_index = np.zeros(self.size, dtype=np.int64)
        chatty = not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0
        t0 = time.time()
        helpers.build_blending_indices(self.dataset_index, self.dataset_sample_index, share, len(datasets),
                                       self.size, chatty)
        print_rank_0(f"> elapsed time for building blendable dataset indices: {time.time() - t0:.2f} (sec)")

    def __len__(self):
        return self.size

    def __getitem__(self, idx):
        if not 0 <= idx < self.size:
            wrapped = idx % self.size
            print(f"WARNING: Got index out of bounds error with index {idx} - taking modulo of index instead "
                  f"({wrapped})")
            idx = wrapped
        component = self.datasets[int(self.dataset_index[idx])]
        item = int(self.dataset_sample_index[idx])
        # a component asked for more items than it holds (rounding of the shares) wraps around as well
        return component[item] if item < len(component) else component[item % len(component)]
