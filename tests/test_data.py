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


def test_index_files_follow_the_documented_byte_layout(tmp_path):
    """Readers accept hand-packed index files of both layouts (the byte layout existing corpora use), and the
    builders emit exactly those bytes."""
    import struct
    docs = [np.array([5, 6, 7], dtype=np.uint16), np.array([9], dtype=np.uint16), np.array([1, 2], dtype=np.uint16)]
    flat = np.concatenate(docs)
    # ---- mmap layout
    pfx = str(tmp_path / "hand_mmap")
    flat.tofile(pfx + ".bin")
    sizes = np.array([3, 1, 2], dtype=np.int32)
    ptrs = np.array([0, 6, 8], dtype=np.int64)
    doc_idx = np.array([0, 2, 3], dtype=np.int64)
    blob = b"MMIDIDX\x00\x00" + struct.pack("<Q", 1) + struct.pack("<B", 8) + struct.pack("<Q", 3) + \
        struct.pack("<Q", 3) + sizes.tobytes() + ptrs.tobytes() + doc_idx.tobytes()
    open(pfx + ".idx", "wb").write(blob)
    ds = indexed_dataset.make_dataset(pfx, "infer", skip_warmup=True)
    assert [list(ds[i]) for i in range(3)] == [[5, 6, 7], [9], [1, 2]] and list(ds.doc_idx) == [0, 2, 3]
    assert [list(a) for a in ds[0:3]] == [[5, 6, 7], [9], [1, 2]] and list(ds.get(0, 1, 2)) == [6, 7]
    b = indexed_dataset.MMapIndexedDatasetBuilder(str(tmp_path / "built.bin"), dtype=np.uint16)
    b.add_items(docs[:2])
    b.end_document()
    b.add_item(docs[2])
    b.end_document()
    b.finalize(str(tmp_path / "built.idx"))
    assert open(tmp_path / "built.idx", "rb").read() == blob
    assert open(tmp_path / "built.bin", "rb").read() == flat.tobytes()
    # ---- legacy layout (int32 items)
    pfx = str(tmp_path / "hand_legacy")
    flat32 = flat.astype(np.int32)
    flat32.tofile(pfx + ".bin")
    i64 = lambda *v: np.array(v, dtype=np.int64).tobytes()
    blob = b"TNTIDX\x00\x00" + struct.pack("<Q", 1) + struct.pack("<QQ", 4, 4) + struct.pack("<QQ", 3, 3) + \
        struct.pack("<Q", 3) + i64(0, 1, 2, 3) + i64(0, 3, 4, 6) + i64(3, 1, 2) + i64(0, 2, 3)
    open(pfx + ".idx", "wb").write(blob)
    assert indexed_dataset.infer_dataset_impl(pfx) == "cached"
    lazy = indexed_dataset.make_dataset(pfx, "lazy")
    assert [list(lazy[i]) for i in range(3)] == [[5, 6, 7], [9], [1, 2]] and [list(a) for a in lazy[1:3]] == [[9], [1, 2]]
    b = indexed_dataset.IndexedDatasetBuilder(str(tmp_path / "built_legacy.bin"), dtype=np.int32)
    for i, d in enumerate(docs):
        b.add_item(d.astype(np.int32))
        if i in (1, 2):
            b.end_document()
    b.finalize(str(tmp_path / "built_legacy.idx"))
    assert open(tmp_path / "built_legacy.idx", "rb").read() == blob


def test_mmap_builder_merge_shifts_document_boundaries(tmp_path):
    rng = np.random.default_rng(3)
    a, b = _docs(rng, 5), _docs(rng, 4)
    pa, pb = _write(tmp_path, a, name="a"), _write(tmp_path, b, name="b")
    m = indexed_dataset.MMapIndexedDatasetBuilder(str(tmp_path / "m.bin"), dtype=np.uint16)
    m.merge_file_(pa)
    m.merge_file_(pb)
    m.finalize(str(tmp_path / "m.idx"))
    ds = indexed_dataset.make_dataset(str(tmp_path / "m"), "mmap", skip_warmup=True)
    assert len(ds) == 9 and list(ds.doc_idx) == list(range(10))
    for i, d in enumerate(a + b):
        assert np.array_equal(ds[i], d)


@pytest.mark.parametrize("pack_impl", ["unpacked", "pack_until_overflow"])
def test_whole_document_items_respect_the_split_and_never_borrow_tokens(tmp_path, pack_impl):
    """`unpacked` / `pack_until_overflow` items are made of whole documents of THEIR split (a split that starts
    at document 30 must not read document 0) and carry no token of the following document."""
    from gpt_neox_b200.data.gpt2_dataset import GPT2Dataset
    rng = np.random.default_rng(5)
    docs = [np.full(int(rng.integers(3, 9)), 100 + i, dtype=np.int32) for i in range(40)]     # doc i is all (100 + i)
    prefix = _write(tmp_path, docs)
    ds = indexed_dataset.make_dataset(prefix, "mmap", skip_warmup=True)
    split = np.arange(30, 40, dtype=np.int32)
    seq = 16
    g = GPT2Dataset("valid", prefix, split, ds, num_samples=12, num_epochs=None, seq_length=seq, seed=1,
                    pack_impl=pack_impl, use_shared_fs=True)
    seen = set()
    for i in range(len(g)):
        item = g[i]["text"]
        assert item.shape == (seq + 1,)
        body = item[item != 0]                                   # zero padding at the end
        ids = sorted(set(int(t) - 100 for t in body))
        assert all(30 <= d < 40 for d in ids)                    # only documents of the split
        assert len(body) == sum(len(docs[d]) for d in ids)       # whole documents, nothing borrowed
        if pack_impl == "unpacked":
            assert len(ids) == 1
        seen.update(ids)
    assert len(seen) >= 5
