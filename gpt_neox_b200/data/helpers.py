"""ctypes binding of ``lib/libneox_data.so`` (csrc/data_helpers.cpp) with the same function names
as the reference's pybind11 ``helpers`` module (megatron/data/helpers.cpp), plus NumPy
restatements used as test oracles."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

_LIB = None
_PATH = Path(__file__).resolve().parent.parent / "lib" / "libneox_data.so"


def compile_helper():
    """Build the shared library if it is missing or stale (the reference runs ``make`` in
    megatron/data at start-up, megatron/data/data_utils.py:809-821)."""
    from ..build import build_data_helpers
    build_data_helpers()


def _lib():
    global _LIB
    if _LIB is None:
        path = os.environ.get("NEOX_DATA_LIB") or str(_PATH)      # override: a sanitizer build of the same sources
        if path == str(_PATH) and not _PATH.exists():
            compile_helper()
        L = C.CDLL(path)
        P, I32, I64, U64, D = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_double
        L.nx_num_samples.argtypes = [I64, I64, I64]
        L.nx_num_samples.restype = I64
        for n in ("nx_build_sample_idx_i32", "nx_build_sample_idx_i64"):
            getattr(L, n).argtypes = [P, P, I64, I64, I64, P]
            getattr(L, n).restype = None
        L.nx_build_blending_indices.argtypes = [P, P, P, I32, I64, I32]
        L.nx_build_blending_indices.restype = None
        L.nx_build_mapping.argtypes = [P, I64, P, I32, U64, I32, D, I32, P]
        L.nx_build_mapping.restype = I64
        L.nx_build_blocks_mapping.argtypes = [P, I64, P, P, I32, U64, I32, I32, I32, P]
        L.nx_build_blocks_mapping.restype = I64
        _LIB = L
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, dtype):
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
    L = _lib()
    n = L.nx_num_samples(seq_length, num_epochs, tokens_per_epoch)
    out = np.empty((n + 1, 2), dtype=dtype)
    fn = L.nx_build_sample_idx_i32 if dtype == np.int32 else L.nx_build_sample_idx_i64
    fn(_p(sizes), _p(doc_idx), seq_length, num_epochs, tokens_per_epoch, _p(out))
    return out


def build_sample_idx_int32(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch):
    return _build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, np.int32)


def build_sample_idx_int64(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch):
    return _build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch, np.int64)


def build_blending_indices(dataset_index, dataset_sample_index, weights, num_datasets, size, verbose):
    assert dataset_index.dtype == np.uint8 and dataset_sample_index.dtype == np.int64
    weights = np.ascontiguousarray(weights, dtype=np.float64)
    _lib().nx_build_blending_indices(_p(dataset_index), _p(dataset_sample_index), _p(weights), int(num_datasets),
                                     int(size), int(bool(verbose)))


def build_mapping(docs, sizes, num_epochs, max_num_samples, max_seq_length, short_seq_prob, seed, verbose=False):
    docs = np.ascontiguousarray(docs, dtype=np.int64)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    L = _lib()
    args = (_p(docs), len(docs), _p(sizes), int(num_epochs), int(max_num_samples), int(max_seq_length),
            float(short_seq_prob), int(seed))
    rows = L.nx_build_mapping(*args, None)
    out = np.empty((rows, 3), dtype=np.int64)
    L.nx_build_mapping(*args, _p(out))
    return out


def build_blocks_mapping(docs, sizes, titles_sizes, num_epochs, max_num_samples, max_seq_length, seed, verbose=False,
                         use_one_sent_blocks=False):
    docs = np.ascontiguousarray(docs, dtype=np.int64)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    titles_sizes = np.ascontiguousarray(titles_sizes, dtype=np.int32)
    L = _lib()
    args = (_p(docs), len(docs), _p(sizes), _p(titles_sizes), int(num_epochs), int(max_num_samples),
            int(max_seq_length), int(seed), int(bool(use_one_sent_blocks)))
    rows = L.nx_build_blocks_mapping(*args, None)
    out = np.empty((rows, 4), dtype=np.int64)
    L.nx_build_blocks_mapping(*args, _p(out))
    return out


# ---------------------------------------------------------------------------- NumPy oracles
def build_sample_idx_numpy(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch):
    """Python restatement (megatron/data/gpt2_dataset.py:427-472) used to test the C++ builder."""
    num_samples = (num_epochs * tokens_per_epoch - 1) // seq_length
    sample_idx = np.zeros([num_samples + 1, 2], dtype=np.int64)
    sample_index, doc_idx_index, doc_offset = 0, 0, 0
    sample_idx[sample_index] = (doc_idx_index, doc_offset)
    sample_index += 1
    while sample_index <= num_samples:
        remaining = seq_length + 1
        while remaining != 0:
            doc_id = doc_idx[doc_idx_index]
            doc_length = sizes[doc_id] - doc_offset
            remaining -= doc_length
            if remaining <= 0:
                doc_offset += remaining + doc_length - 1
                remaining = 0
            else:
                doc_idx_index += 1
                doc_offset = 0
        sample_idx[sample_index] = (doc_idx_index, doc_offset)
        sample_index += 1
    return sample_idx


def build_blending_indices_numpy(weights, size):
    n = len(weights)
    di = np.zeros(size, dtype=np.uint8)
    dsi = np.zeros(size, dtype=np.int64)
    cur = np.zeros(n, dtype=np.int64)
    for s in range(size):
        want = max(float(s), 1.0)
        err = np.asarray(weights, dtype=np.float64) * want - cur
        b = int(np.argmax(err))
        di[s], dsi[s] = b, cur[b]
        cur[b] += 1
    return di, dsi
