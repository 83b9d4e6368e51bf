"""GPT dataset over an indexed token file (megatron/data/gpt2_dataset.py:29-482): every item is
``seq_length + 1`` tokens cut from the shuffled, concatenated document stream (``packed``), or whole
documents packed until they overflow (``pack_until_overflow``), or one document per item
(``unpacked``); optional parallel label / reward / reference-logprob streams.  The three index
arrays (doc_idx, sample_idx, shuffle_idx) are built once by rank 0, cached as ``.npy`` next to the
data and memory-mapped by everyone."""
from __future__ import annotations

import os
import time

import numpy as np
import torch
import torch.distributed as dist

from .. import parallel as mpu
from ..utils.common import print_rank_0
from . import helpers


class GPT2Dataset(torch.utils.data.Dataset):
    def __init__(self, name, data_prefix, documents, indexed_dataset, num_samples, num_epochs, seq_length, seed,
                 pack_impl="packed", allow_chopped=True, build_index_mappings=True, use_shared_fs=True,
                 label_dataset=None, reward_dataset=None, ref_dataset=None):
        self.name, self.pack_impl, self.allow_chopped = name, pack_impl, allow_chopped
        self.indexed_dataset = indexed_dataset
        self.label_dataset, self.reward_dataset, self.ref_dataset = label_dataset, reward_dataset, ref_dataset
        self.seq_length = seq_length
        assert self.reward_dataset is None or pack_impl == "unpacked", \
            "Reward dataset only supported with unpacked data."
        assert np.min(documents) >= 0
        assert np.max(documents) < indexed_dataset.sizes.shape[0]
        if build_index_mappings:
            self.doc_idx, self.sample_idx, self.shuffle_idx = _build_index_mappings(
                self.name, data_prefix, documents, self.indexed_dataset.sizes, self.label_dataset, num_samples,
                num_epochs, seq_length, seed, self.pack_impl, use_shared_fs=use_shared_fs,
                allow_chopped=self.allow_chopped)
            self.shuffle_idx_len = self.shuffle_idx.shape[0] - 1
            self.sample_idx_len = self.sample_idx.shape[0] - 1
            if self.shuffle_idx_len != self.sample_idx_len - 1:
                print(f"WARNING: shuffle index length ({self.shuffle_idx_len}) is not equal to sample index length "
                      f"({self.sample_idx_len})")

    def __len__(self):
        return min(self.shuffle_idx_len, self.sample_idx_len)

    def _span(self, dataset, first_doc, last_doc, off_first, off_last, is_reward, lengths):
        """Concatenate the pieces of one stream between (first_doc, off_first) and (last_doc, off_last).
        A reward stream repeats each document's scalar over that document's token count."""
        if first_doc == last_doc:
            if is_reward:
                rw = dataset.get(self.doc_idx[first_doc])
                return np.full(lengths[0], rw[0]), lengths
            piece = dataset.get(self.doc_idx[first_doc], offset=off_first, length=off_last - off_first + 1)
            return piece, [len(piece)]
        docs = list(range(first_doc, last_doc + 1))
        pieces, out_lengths = [], []
        for j, d in enumerate(docs):
            if is_reward:
                rw = dataset.get(self.doc_idx[d])
                pieces.append(np.full(lengths[j], rw[0]))
                continue
            if j == 0:
                p = dataset.get(self.doc_idx[d], offset=off_first)
            elif j == len(docs) - 1:
                p = dataset.get(self.doc_idx[d], length=off_last + 1)
            else:
                p = dataset.get(self.doc_idx[d])
            pieces.append(p)
            out_lengths.append(len(p))
        return np.concatenate(pieces), (lengths if is_reward else out_lengths)

    def _whole_docs(self, dataset, first_doc, last_doc, is_reward, lengths):
        """Documents [first_doc, last_doc) in full, concatenated (the unpacked and pack-until-overflow items: an
        item never borrows a token from the document after it)."""
        pieces, out_lengths = [], []
        for j, d in enumerate(range(first_doc, last_doc)):
            if is_reward:
                pieces.append(np.full(lengths[j], dataset.get(self.doc_idx[d])[0]))
            else:
                pieces.append(dataset.get(self.doc_idx[d]))
                out_lengths.append(len(pieces[-1]))
        return np.concatenate(pieces), (lengths if is_reward else out_lengths)

    def __getitem__(self, idx):
        asked = idx
        try:
            idx = self.shuffle_idx[idx]
            first_doc, off_first = self.sample_idx[idx]
            last_doc, off_last = self.sample_idx[idx + 1]
            streams = [("text", self.indexed_dataset, np.int64)]
            if self.label_dataset is not None:
                streams.append(("label", self.label_dataset, np.int64))
            if self.reward_dataset is not None:
                streams.append(("reward", self.reward_dataset, np.float32))
            if self.ref_dataset is not None:
                streams.append(("ref", self.ref_dataset, np.float32))
            ret, lengths = {}, []
            for key, ds, dt in streams:
                if self.pack_impl == "packed":
                    sample, lengths = self._span(ds, int(first_doc), int(last_doc), int(off_first), int(off_last),
                                                 key == "reward", lengths)
                else:
                    sample, lengths = self._whole_docs(ds, int(first_doc), int(last_doc), key == "reward", lengths)
                want = self.seq_length + 1
                if len(sample) < want:
                    sample = np.pad(sample, (0, want - len(sample)), mode="constant",
                                    constant_values=-100 if key == "label" else 0)
                elif len(sample) > want:
                    sample = sample[:want]
                ret[key] = np.array(sample, dtype=dt)
            return ret
        except IndexError as err:
            new_idx = int(asked) % len(self)
            if new_idx == asked:
                raise                   # already in range: a real indexing fault, not a wrap-around request
            print(f"WARNING: Got index out of bounds error with index {asked} - taking modulo of index instead "
                  f"({new_idx}), error: {err}")
            return self[new_idx]


def _num_tokens(documents, sizes):
    return int(np.sum(sizes[documents]))


def _num_epochs(tokens_per_epoch, seq_length, num_samples):
    """Smallest epoch count whose token stream yields ``num_samples`` items (one token is shared
    between neighbouring items)."""
    num_epochs, total_tokens = 0, 0
    while True:
        num_epochs += 1
        total_tokens += tokens_per_epoch
        if ((total_tokens - 1) // seq_length) >= num_samples:
            return num_epochs


def _build_doc_idx(documents, num_epochs, np_rng):
    doc_idx = np.mgrid[0:num_epochs, 0: len(documents)][1]
    doc_idx[:] = documents
    doc_idx = doc_idx.reshape(-1).astype(np.int32)
    np_rng.shuffle(doc_idx)
    return doc_idx


def _build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch):
    return helpers.build_sample_idx_numpy(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch)


def _build_shuffle_idx(size, np_rng):
    dtype_ = np.uint32 if size < (np.iinfo(np.uint32).max - 1) else np.int64
    shuffle_idx = np.arange(start=0, stop=size, step=1, dtype=dtype_)
    np_rng.shuffle(shuffle_idx)
    return shuffle_idx


def _build_index_mappings(name, data_prefix, documents, sizes, label_dataset, num_samples, num_epochs, seq_length,
                          seed, packing_impl, use_shared_fs=True, allow_chopped=True):
    tokens_per_epoch = _num_tokens(documents, sizes)
    if not num_epochs:
        num_epochs = _num_epochs(tokens_per_epoch, seq_length, num_samples)
    np_rng = np.random.RandomState(seed=seed)
    base = f"{data_prefix}_{name}_indexmap_{num_samples}ns_{seq_length}sl_{seed}s_{packing_impl}pi"
    if not allow_chopped:
        base += "_ac"
    doc_idx_filename = base + "_doc_idx.npy"
    sample_idx_filename = base + "_sample_idx.npy"
    shuffle_idx_filename = base + "_shuffle_idx.npy"
    rank = dist.get_rank() if dist.is_initialized() else 0
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    should_build = rank == 0 if use_shared_fs else local_rank == 0
    if should_build and not all(os.path.isfile(f) for f in (doc_idx_filename, sample_idx_filename,
                                                            shuffle_idx_filename)):
        print_rank_0(" > WARNING: could not find index map files, building the indices on rank 0 ...")
        start_time = time.time()
        if packing_impl == "packed":
            doc_idx = _build_doc_idx(documents, num_epochs, np_rng)
            np.save(doc_idx_filename, doc_idx, allow_pickle=True)
            assert doc_idx.dtype == np.int32 and sizes.dtype == np.int32
            n_samples = (num_epochs * tokens_per_epoch - 1) / seq_length
            if 2 * (n_samples + 1) < np.iinfo(np.int32).max:
                sample_idx = helpers.build_sample_idx_int32(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch)
            else:
                sample_idx = helpers.build_sample_idx_int64(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch)
            np.save(sample_idx_filename, sample_idx, allow_pickle=True)
            shuffle_idx = _build_shuffle_idx(sample_idx.shape[0] - 1, np_rng)
            np.save(shuffle_idx_filename, shuffle_idx, allow_pickle=True)
        elif packing_impl == "pack_until_overflow":
            shuffle_idx = np.arange(num_samples)
            np_rng.shuffle(shuffle_idx)
            sample_idx, doc_idx = [], []
            order = np.arange(len(documents))
            np_rng.shuffle(order)
            running, cur = 0, 0
            while len(sample_idx) < num_samples:
                d = int(documents[order[cur]])          # document id in the indexed dataset (splits start anywhere)
                skip = (not allow_chopped and sizes[d] > seq_length + 1) or \
                       (label_dataset is not None and np.all(label_dataset.get(d)[: seq_length + 1] == -100))
                if not skip:
                    doc_length = sizes[d]
                    if running == 0:
                        sample_idx.append(np.array([len(doc_idx), 0]))
                        running += doc_length
                    elif running + doc_length > (seq_length + 1):
                        running = doc_length
                        sample_idx.append(np.array([len(doc_idx), 0]))
                    else:
                        running += doc_length
                    doc_idx.append(d)
                cur += 1
                if cur == len(documents):
                    cur = 0
                    np_rng.shuffle(order)
            sample_idx.append(np.array([len(doc_idx), 0]))
            np.save(doc_idx_filename, doc_idx, allow_pickle=True)
            np.save(sample_idx_filename, sample_idx, allow_pickle=True)
            np.save(shuffle_idx_filename, shuffle_idx, allow_pickle=True)
        elif packing_impl == "unpacked":
            shuffle_idx = np.arange(num_samples)
            np_rng.shuffle(shuffle_idx)
            sample_idx = np.zeros((num_samples + 1, 2), dtype=np.int64)
            sample_idx[:, 0] = np.arange(num_samples + 1)
            doc_idx, at, examined = [], 0, 0
            while len(doc_idx) <= num_samples:
                d = int(documents[at])                  # document id in the indexed dataset (splits start anywhere)
                skip = (not allow_chopped and sizes[d] > seq_length + 1) or \
                       (label_dataset is not None and np.all(label_dataset.get(d)[:seq_length] == -100))
                if not skip:
                    doc_idx.append(d)
                at = (at + 1) % len(documents)
                examined += 1
                if examined == len(documents) and not doc_idx:
                    raise ValueError(f"{name}: every document is either longer than seq_length + 1 (allow_chopped "
                                     f"is off) or fully masked by its labels")
            np.save(doc_idx_filename, doc_idx, allow_pickle=True)
            np.save(sample_idx_filename, sample_idx, allow_pickle=True)
            np.save(shuffle_idx_filename, shuffle_idx, allow_pickle=True)
        print_rank_0(" > elapsed time to build and save index mappings (seconds): {:4f}".format(
            time.time() - start_time))
    # everyone waits for the builder (an all-reduce over the IO group serves as the barrier)
    if dist.is_initialized():
        counts = torch.ones(1, dtype=torch.long, device="cuda" if dist.get_backend() == "nccl" else "cpu")
        dist.all_reduce(counts, group=mpu.get_io_parallel_group())
        dist.barrier()
    start_time = time.time()
    doc_idx = np.load(doc_idx_filename, allow_pickle=True, mmap_mode="r")
    sample_idx = np.load(sample_idx_filename, allow_pickle=True, mmap_mode="r")
    shuffle_idx = np.load(shuffle_idx_filename, allow_pickle=True, mmap_mode="r")
    print_rank_0("    loaded indexed file in {:3.3f} seconds".format(time.time() - start_time))
    print_rank_0("    total number of samples: {}".format(shuffle_idx.shape[0] + 1))
    print_rank_0("    total number of epochs: {}".format(num_epochs))
    return doc_idx, sample_idx, shuffle_idx
