"""Data path: native index builders against their NumPy restatements, indexed-dataset round trips, sample
boundaries of the packed GPT-2 dataset, blending proportions, resumable sampling."""
import numpy as np
import pytest
import torch

from common import ROOT  # noqa: F401
from gpt_neox_b200.data import helpers, indexed_dataset


def _docs(rng, n=50, lo=1, hi=40):
    return [rng.integers(1, 1000, size=int(rng.integers(lo, hi))).astype(np.int32) for _ in range(n)]


def _write(tmp_path, docs, impl="mmap", name="ds"):
    prefix = str(tmp_path / name)
    b = indexed_dataset.make_builder(prefix + ".bin", impl=impl, vocab_size=1000)
    for d in docs:
        b.add_item(np.asarray(d, dtype=b.dtype))
        b.end_document()
    b.finalize(prefix + ".idx")
    return prefix


@pytest.mark.parametrize("impl", ["mmap", "cached"])
def test_indexed_dataset_round_trip(tmp_path, impl):
    rng = np.random.default_rng(0)
    docs = _docs(rng)
    prefix = _write(tmp_path, docs, impl)
    assert indexed_dataset.infer_dataset_impl(prefix) == impl
    ds = indexed_dataset.make_dataset(prefix, impl, skip_warmup=True)
    assert len(ds) == len(docs)
    if impl == "cached":
        ds.prefetch(range(len(ds)))           # the cached reader serves only what was prefetched
    for i in (0, 7, len(docs) - 1):
        assert np.array_equal(np.asarray(ds[i]), docs[i])
    if impl == "mmap":
        assert np.array_equal(ds.get(3, offset=1, length=2), docs[3][1:3]) or len(docs[3]) < 3
        assert np.array_equal(np.asarray(ds.sizes), [len(d) for d in docs])


@pytest.mark.parametrize("seq_length,epochs", [(16, 1), (7, 3), (64, 2)])
def test_native_sample_index_matches_numpy(seq_length, epochs):
    rng = np.random.default_rng(1)
    sizes = rng.integers(1, 50, size=200).astype(np.int32)
    doc_idx = np.concatenate([rng.permutation(200) for _ in range(epochs)]).astype(np.int32)
    tpe = int(sizes.sum())
    want = helpers.build_sample_idx_numpy(sizes, doc_idx, seq_length, epochs, tpe)
    got32 = helpers.build_sample_idx_int32(sizes, doc_idx, seq_length, epochs, tpe)
    got64 = helpers.build_sample_idx_int64(sizes, doc_idx.astype(np.int64), seq_length, epochs, tpe)
    assert np.array_equal(got32, want) and np.array_equal(got64, want)


def test_native_blending_matches_numpy_and_weights():
    w = np.array([0.5, 0.3, 0.2])
    size = 1000
    di = np.zeros(size, dtype=np.uint8)
    dsi = np.zeros(size, dtype=np.int64)
    helpers.build_blending_indices(di, dsi, w, 3, size, False)
    wdi, wdsi = helpers.build_blending_indices_numpy(w, size)
    assert np.array_equal(di, wdi) and np.array_equal(dsi, wdsi)
    frac = np.bincount(di, minlength=3) / size
    assert np.allclose(frac, w, atol=0.01)
    for k in range(3):
        assert np.array_equal(dsi[di == k], np.arange((di == k).sum()))      # each source is read in order


def test_gpt2_dataset_samples_are_contiguous_token_windows(tmp_path):
    from gpt_neox_b200.data.gpt2_dataset import GPT2Dataset
    rng = np.random.default_rng(2)
    docs = _docs(rng, n=30, lo=5, hi=60)
    prefix = _write(tmp_path, docs)
    ds = indexed_dataset.make_dataset(prefix, "mmap", skip_warmup=True)
    seq = 16
    g = GPT2Dataset("t", prefix, np.arange(len(docs), dtype=np.int32), ds, num_samples=40, num_epochs=None,
                    seq_length=seq, seed=3, use_shared_fs=False)
    assert len(g) >= 40
    stream = np.concatenate([docs[i] for i in g.doc_idx])
    for i in range(len(g)):
        x = g[i]["text"]
        assert x.shape == (seq + 1,)
        j = int(g.shuffle_idx[i])
        assert np.array_equal(x, stream[j * seq: j * seq + seq + 1])        # sample j = tokens [j*s, j*s + s]
    # deterministic in the seed
    g2 = GPT2Dataset("t", prefix, np.arange(len(docs), dtype=np.int32), ds, num_samples=40, num_epochs=None,
                     seq_length=seq, seed=3, use_shared_fs=False)
    assert np.array_equal(g2[5]["text"], g[5]["text"])


def test_batch_sampler_shards_and_resumes():
    from gpt_neox_b200.data.samplers import DistributedBatchSampler
    from torch.utils.data import SequentialSampler
    data = list(range(64))
    seen = []
    for rank in range(2):
        s = DistributedBatchSampler(SequentialSampler(data), batch_size=8, drop_last=True, rank=rank, world_size=2)
        seen.append([b for b in s])
    assert seen[0][0] == [0, 1, 2, 3] and seen[1][0] == [4, 5, 6, 7]
    assert sorted(sum(seen[0] + seen[1], [])) == data
    s = DistributedBatchSampler(SequentialSampler(data), batch_size=8, drop_last=True, rank=0, world_size=2)
    s.start_iter = 3                                                         # resume after 3 global batches
    assert next(iter(s)) == [24, 25, 26, 27]
