"""Paired (chosen / rejected) dataset for preference learning: DPO and reward-model training
(megatron/data/pairwise_dataset.py:29-186).

Document ``i`` of the positive stream is paired with document ``i`` of the negative stream; a sample is one
pair (never packed), cut or padded to ``seq_length + 1`` tokens.  Optional label streams (-100 = not scored)
and reference log-prob streams ride along with identical cutting.  The sample order is a seeded shuffle of
the usable documents, repeated for as many epochs as ``num_samples`` needs; it is recomputed from the seed
(cheap: one permutation per epoch), so no index cache files are written.
"""
from __future__ import annotations

import numpy as np
import torch


class PairwiseDataset(torch.utils.data.Dataset):
    def __init__(self, name, pos_data_prefix, documents, pos_indexed_dataset, neg_indexed_dataset, num_samples,
                 seq_length, seed, pack_impl="unpacked", build_index_mappings=True, use_shared_fs=True,
                 pos_label_dataset=None, pos_ref_dataset=None, neg_label_dataset=None, neg_ref_dataset=None,
                 allow_chopped=True):
        self.name = name
        self.pos_indexed_dataset, self.neg_indexed_dataset = pos_indexed_dataset, neg_indexed_dataset
        self.pos_label_dataset, self.neg_label_dataset = pos_label_dataset, neg_label_dataset
        self.pos_ref_dataset, self.neg_ref_dataset = pos_ref_dataset, neg_ref_dataset
        self.pack_impl, self.seq_length = pack_impl, seq_length
        documents = np.asarray(documents)
        assert np.min(documents) >= 0
        assert (neg_label_dataset is None) == (pos_label_dataset is None), \
            "Label datasets must be both None or both not None"
        assert np.max(documents) < pos_indexed_dataset.sizes.shape[0]
        assert pos_indexed_dataset.sizes.shape[0] == neg_indexed_dataset.sizes.shape[0]
        assert pack_impl != "packed", "Packed implementation not supported for pairwise dataset"
        if not allow_chopped:
            longest = np.maximum(np.asarray(pos_indexed_dataset.sizes)[documents],
                                 np.asarray(neg_indexed_dataset.sizes)[documents])
            documents = documents[longest <= seq_length + 1]
        self.documents = documents
        self.order = np.zeros(0, dtype=np.int64)
        if build_index_mappings and len(documents):
            rng = np.random.RandomState(seed)
            epochs = max(1, -(-int(num_samples) // len(documents)))
            self.order = np.concatenate([rng.permutation(documents) for _ in range(epochs)]).astype(np.int64)

    def __len__(self):
        return len(self.order)

    def _fit(self, arr, pad, dtype):
        n = self.seq_length + 1
        arr = np.asarray(arr)[:n]
        if len(arr) < n:
            arr = np.pad(arr, (0, n - len(arr)), mode="constant", constant_values=pad)
        return np.array(arr, dtype=dtype)

    def __getitem__(self, idx):
        if idx >= len(self.order):
            new = idx % len(self.order)
            print(f"WARNING: Got index out of bounds error with index {idx} - taking modulo of index instead ({new})")
            idx = new
        doc = int(self.order[idx])
        ret = {"pos": self._fit(self.pos_indexed_dataset.get(doc), 0, np.int64),
               "neg": self._fit(self.neg_indexed_dataset.get(doc), 0, np.int64)}
        if self.pos_label_dataset is not None:
            ret["pos_label"] = self._fit(self.pos_label_dataset.get(doc), -100, np.int64)
            ret["neg_label"] = self._fit(self.neg_label_dataset.get(doc), -100, np.int64)
        if self.pos_ref_dataset is not None:
            ret["pos_ref"] = self._fit(self.pos_ref_dataset.get(doc), 0, np.float32)
            ret["neg_ref"] = self._fit(self.neg_ref_dataset.get(doc), 0, np.float32)
        return ret
