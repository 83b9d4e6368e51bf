"""Token datasets on disk: ``<prefix>.bin`` holds the raw token stream, ``<prefix>.idx`` describes it.

Two index layouts are read and written, byte-compatible with the files the reference produces
(megatron/data/indexed_dataset.py) so that existing tokenised corpora load unchanged:

``mmap`` (magic ``MMIDIDX\\0\\0``)
    ``<Q version=1> <B dtype code> <Q n_sequences> <Q n_doc_boundaries>`` followed by three arrays:
    int32 sequence lengths, int64 byte offsets of every sequence in the .bin file, int64 document boundaries
    (indices into the sequence list; first entry 0).  The .bin file is mapped, never read eagerly.

``cached`` / ``lazy`` (magic ``TNTIDX\\0\\0``, the older layout)
    ``<Q version=1> <Q dtype code> <Q element size> <Q n_items> <Q n_dims_total> <Q n_doc_boundaries>`` followed by
    four int64 arrays: per-item offsets into the dims array, per-item element offsets into the .bin file, the
    dims of every item, the document boundaries.

The module is organised as plain records + functions for the two index layouts (``MMapIndex``, ``LegacyIndex``),
reader classes over them and one writer base class; the reader / builder class names and methods are the ones
the rest of the data pipeline (and the reference's tools) use.
"""
from __future__ import annotations

import os
import shutil
import struct
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence

import numpy as np
import torch

MMAP_MAGIC = b"MMIDIDX\x00\x00"
LEGACY_MAGIC = b"TNTIDX\x00\x00"

# dtype codes stored in the index files
dtypes = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64,
          8: np.uint16, 9: np.uint32, 10: np.uint64}
_CODE_OF = {np.dtype(v): k for k, v in dtypes.items()}


def code(dtype) -> int:
    try:
        return _CODE_OF[np.dtype(dtype)]
    except KeyError:
        raise ValueError(f"no index code for dtype {dtype}") from None


def best_fitting_dtype(vocab_size: Optional[int] = None):
    """uint16 when every token id fits, int32 otherwise."""
    return np.uint16 if (vocab_size is not None and vocab_size < 65500) else np.int32


def index_file_path(prefix: str) -> str:
    return prefix + ".idx"


def data_file_path(prefix: str) -> str:
    return prefix + ".bin"


def _both_files(prefix: str) -> bool:
    return os.path.exists(index_file_path(prefix)) and os.path.exists(data_file_path(prefix))


def infer_dataset_impl(prefix: str) -> Optional[str]:
    """``"mmap"`` / ``"cached"`` from the index magic; None when the files are missing or unknown."""
    if not _both_files(prefix):
        print(f"Dataset does not exist: {prefix}")
        print("Path should be a basename that both .idx and .bin can be appended to get full filenames.")
        return None
    with open(index_file_path(prefix), "rb") as f:
        head = f.read(9)
    if head.startswith(LEGACY_MAGIC):
        return "cached"
    if head == MMAP_MAGIC:
        return "mmap"
    return None


def make_dataset(prefix: str, impl: str, skip_warmup: bool = False):
    if not _both_files(prefix):
        print(f"Dataset does not exist: {prefix}")
        print("Path should be a basename that both .idx and .bin can be appended to get full filenames.")
        return None
    if impl == "infer":
        impl = infer_dataset_impl(prefix)
    readers = {"lazy": IndexedDataset, "cached": IndexedCachedDataset}
    if impl in readers:
        return readers[impl](prefix)
    if impl == "mmap":
        return MMapIndexedDataset(prefix, skip_warmup)
    print(f"Unknown dataset implementation: {impl}")
    return None


def make_builder(out_file: str, impl: str, vocab_size: Optional[int] = None):
    if impl == "mmap":
        return MMapIndexedDatasetBuilder(out_file, dtype=best_fitting_dtype(vocab_size))
    return IndexedDatasetBuilder(out_file)


def dataset_exists(prefix: str, impl: str) -> bool:
    return _both_files(prefix)


def create_doc_idx(sizes: Sequence[int]) -> List[int]:
    """Document boundaries of a stream in which an empty sequence ends a document."""
    return [0] + [i + 1 for i, n in enumerate(sizes) if n == 0]


# ------------------------------------------------------------------------------------------ legacy layout
@dataclass
class LegacyIndex:
    dtype: type
    element_size: int
    dim_offsets: np.ndarray     # [n + 1]
    data_offsets: np.ndarray    # [n + 1], in elements
    sizes: np.ndarray           # dims of every item, concatenated
    doc_idx: np.ndarray

    @property
    def n(self) -> int:
        return len(self.data_offsets) - 1

    @classmethod
    def load(cls, path: str) -> "LegacyIndex":
        with open(path, "rb") as f:
            if f.read(8) != LEGACY_MAGIC:
                raise ValueError("Index file doesn't match expected format. Make sure that --dataset-impl is "
                                 "configured properly.")
            version, dcode, esize, n, n_dims, n_docs = struct.unpack("<6Q", f.read(48))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            take = lambda k: np.fromfile(f, dtype=np.int64, count=k)
            return cls(dtypes[dcode], int(esize), take(n + 1), take(n + 1), take(n_dims), take(n_docs))

    def store(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(LEGACY_MAGIC)
            f.write(struct.pack("<6Q", 1, code(self.dtype), self.element_size, self.n, len(self.sizes),
                                len(self.doc_idx)))
            for arr in (self.dim_offsets, self.data_offsets, self.sizes, self.doc_idx):
                f.write(np.asarray(arr, dtype=np.int64).tobytes(order="C"))

    def shape_of(self, i: int):
        return tuple(int(d) for d in self.sizes[self.dim_offsets[i]:self.dim_offsets[i + 1]])


class IndexedDataset(torch.utils.data.Dataset):
    """Legacy layout, every item read from the .bin file when asked for ("lazy")."""

    supports_prefetch = False

    def __init__(self, path: str):
        super().__init__()
        self.path = path
        self._index = LegacyIndex.load(index_file_path(path))
        self._fh = None

    # the fields the dataset tools look at
    dtype = property(lambda self: self._index.dtype)
    sizes = property(lambda self: self._index.sizes)
    doc_idx = property(lambda self: self._index.doc_idx)
    data_offsets = property(lambda self: self._index.data_offsets)
    dim_offsets = property(lambda self: self._index.dim_offsets)
    element_size = property(lambda self: self._index.element_size)

    def __len__(self):
        return self._index.n

    def _check(self, i: int) -> int:
        if not -len(self) <= i < len(self):
            raise IndexError("index out of range")
        return i % len(self)

    def _read_elements(self, first: int, count: int) -> np.ndarray:
        if self._fh is None:
            self._fh = open(data_file_path(self.path), "rb", buffering=0)
        self._fh.seek(int(first) * self._index.element_size)
        out = np.empty(int(count), dtype=self._index.dtype)
        self._fh.readinto(out)
        return out

    def _item(self, i: int) -> np.ndarray:
        lo, hi = self._index.data_offsets[i], self._index.data_offsets[i + 1]
        return self._read_elements(lo, hi - lo).reshape(self._index.shape_of(i))

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            if step != 1:
                raise ValueError("Slices into indexed_dataset must be contiguous")
            if stop <= start:
                return []
            off = self._index.data_offsets
            flat = self._read_elements(off[start], off[stop] - off[start])       # one read for the whole range
            cuts = (off[start + 1:stop] - off[start]).astype(np.int64)
            return [p.reshape(self._index.shape_of(start + k)) for k, p in enumerate(np.split(flat, cuts))]
        return self._item(self._check(int(idx)))

    def num_tokens(self, i):
        return self._index.sizes[i]

    size = num_tokens

    @property
    def supports_prefetch(self):
        return False          # IndexedCachedDataset overrides this

    @staticmethod
    def exists(prefix):
        return _both_files(prefix)

    def __del__(self):
        if getattr(self, "_fh", None) is not None:
            self._fh.close()


class IndexedCachedDataset(IndexedDataset):
    """Legacy layout served from one in-memory arena that ``prefetch`` fills for a chosen set of items."""

    supports_prefetch = True

    def __init__(self, path: str):
        super().__init__(path)
        self._arena = np.empty(0, dtype=self._index.dtype)
        self._where = {}            # item -> first element in the arena

    @property
    def supports_prefetch(self):
        return True

    def prefetch(self, indices: Iterable[int]):
        wanted = sorted({int(i) for i in indices})
        if all(i in self._where for i in wanted):
            return
        off = self._index.data_offsets
        lengths = [int(off[i + 1] - off[i]) for i in wanted]
        self._arena = np.empty(sum(lengths), dtype=self._index.dtype)
        self._where, at = {}, 0
        for i, n in zip(wanted, lengths):
            self._arena[at:at + n] = self._read_elements(off[i], n)
            self._where[i] = at
            at += n
        if self._fh is not None:        # everything needed is in memory now
            self._fh.close()
            self._fh = None

    def _item(self, i: int) -> np.ndarray:
        if i not in self._where:
            raise KeyError(f"item {i} was not prefetched")
        n = int(self._index.data_offsets[i + 1] - self._index.data_offsets[i])
        at = self._where[i]
        return self._arena[at:at + n].copy().reshape(self._index.shape_of(i))

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return [self._item(i) for i in range(*idx.indices(len(self)))]
        return self._item(self._check(int(idx)))


# ------------------------------------------------------------------------------------------ mmap layout
@dataclass
class MMapIndex:
    dtype: type
    sizes: np.ndarray        # int32 [n]
    pointers: np.ndarray     # int64 [n], byte offsets
    doc_idx: np.ndarray      # int64 [n_docs]

    _HEADER = struct.Struct("<QBQQ")

    @classmethod
    def load(cls, path: str, warm: bool = False) -> "MMapIndex":
        with open(path, "rb") as f:
            if f.read(9) != MMAP_MAGIC:
                raise ValueError("Index file doesn't match expected format. Make sure that --dataset-impl is "
                                 "configured properly.")
            version, dcode, n, n_docs = cls._HEADER.unpack(f.read(cls._HEADER.size))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            base = f.tell()
        if warm:
            _touch_file(path)
        raw = np.memmap(path, mode="r", order="C")
        sizes = np.frombuffer(raw, dtype=np.int32, count=n, offset=base)
        pointers = np.frombuffer(raw, dtype=np.int64, count=n, offset=base + sizes.nbytes)
        doc_idx = np.frombuffer(raw, dtype=np.int64, count=n_docs, offset=base + sizes.nbytes + pointers.nbytes)
        idx = cls(dtypes[dcode], sizes, pointers, doc_idx)
        idx._raw = raw          # keeps the mapping alive
        return idx

    @staticmethod
    def store(path: str, dtype, sizes: Sequence[int], doc_idx: Sequence[int]) -> None:
        lengths = np.asarray(sizes, dtype=np.int64)
        pointers = np.zeros(len(lengths), dtype=np.int64)
        if len(lengths) > 1:
            np.cumsum(lengths[:-1] * np.dtype(dtype).itemsize, out=pointers[1:])
        with open(path, "wb") as f:
            f.write(MMAP_MAGIC)
            f.write(MMapIndex._HEADER.pack(1, code(dtype), len(lengths), len(doc_idx)))
            f.write(lengths.astype(np.int32).tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(doc_idx, dtype=np.int64).tobytes(order="C"))


def _touch_file(path: str, chunk: int = 100 << 20) -> None:
    """Read the file once so that the page cache holds it before the first random accesses."""
    with open(path, "rb") as f:
        while f.read(chunk):
            pass


class MMapIndexedDataset(torch.utils.data.Dataset):
    """Memory-mapped token store: ``ds[i]`` / ``ds.get(i, offset, length)`` are views into the mapped .bin."""

    supports_prefetch = False

    def __init__(self, path: str, skip_warmup: bool = False):
        super().__init__()
        self._open(path, skip_warmup)

    def _open(self, path: str, skip_warmup: bool):
        self._path = path
        self._index = MMapIndex.load(index_file_path(path), warm=not skip_warmup)
        if not skip_warmup:
            _touch_file(data_file_path(path))
        self._tokens = np.memmap(data_file_path(path), mode="r", order="C")
        # a user-supplied document index (dataset tools re-partition documents) overrides the stored one
        self._doc_idx_override = None

    # pickling (DataLoader workers) re-opens the maps instead of copying them
    def __getstate__(self):
        return self._path

    def __setstate__(self, path):
        self._open(path, skip_warmup=True)

    def __len__(self):
        return len(self._index.sizes)

    @property
    def sizes(self):
        return self._index.sizes

    def size(self, index):
        return self._index.sizes[index]

    def num_tokens(self, index):
        return self._index.sizes[index]

    @property
    def supports_prefetch(self):
        return False          # the file is memory-mapped: the page cache does the prefetching

    @property
    def dtype(self):
        return self._index.dtype

    @property
    def doc_idx(self):
        return self._index.doc_idx if self._doc_idx_override is None else self._doc_idx_override

    def get_doc_idx(self):
        return self.doc_idx

    def set_doc_idx(self, doc_idx_):
        self._doc_idx_override = doc_idx_

    def _view(self, byte_offset: int, count: int) -> np.ndarray:
        return np.frombuffer(self._tokens, dtype=self._index.dtype, count=int(count), offset=int(byte_offset))

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        """Tokens ``[offset, offset + length)`` of sequence ``idx`` (to its end when ``length`` is None)."""
        n = int(self._index.sizes[idx]) - offset if length is None else length
        start = int(self._index.pointers[idx]) + offset * np.dtype(self._index.dtype).itemsize
        return self._view(start, n)

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            if step != 1:
                raise ValueError("Slices into indexed_dataset must be contiguous")
            if stop <= start:
                return []
            lengths = self._index.sizes[start:stop]
            flat = self._view(self._index.pointers[start], int(lengths.sum()))
            return np.split(flat, np.cumsum(lengths[:-1], dtype=np.int64))
        i = int(idx)
        if not -len(self) <= i < len(self):
            raise IndexError("index out of range")
        return self.get(i % len(self))

    @staticmethod
    def exists(prefix):
        return _both_files(prefix)

    def __del__(self):
        tok = getattr(self, "_tokens", None)
        if tok is not None and getattr(tok, "_mmap", None) is not None:
            tok._mmap.close()
            self._tokens = None


# ------------------------------------------------------------------------------------------ writers
class _StreamWriter:
    """Appends items to a .bin file and keeps the bookkeeping common to both index layouts."""

    def __init__(self, out_file: str, dtype):
        self._bin = open(out_file, "wb")
        self._dtype = np.dtype(dtype).type
        self._doc_idx = [0]

    @property
    def dtype(self):
        return self._dtype

    def _append_bytes(self, arr: np.ndarray) -> int:
        return self._bin.write(np.ascontiguousarray(arr, dtype=self._dtype).tobytes(order="C"))

    def _append_file(self, prefix: str) -> None:
        with open(data_file_path(prefix), "rb") as src:
            shutil.copyfileobj(src, self._bin)


class IndexedDatasetBuilder(_StreamWriter):
    """Writer of the legacy layout (items may have any shape)."""

    def __init__(self, out_file: str, dtype=np.int32):
        super().__init__(out_file, dtype)
        self._data_offsets, self._dim_offsets, self._dims = [0], [0], []

    def add_item(self, arr: np.ndarray):
        if not (isinstance(arr, np.ndarray) and arr.dtype == self._dtype):
            raise TypeError(f"add_item expects a numpy array of {self._dtype}, got {type(arr)} {getattr(arr, 'dtype', '')}")
        self._append_bytes(arr)
        self._data_offsets.append(self._data_offsets[-1] + arr.size)
        self._dims.extend(arr.shape)
        self._dim_offsets.append(self._dim_offsets[-1] + arr.ndim)

    def end_document(self):
        self._doc_idx.append(len(self._dims))

    def merge_file_(self, other_prefix: str):
        other = LegacyIndex.load(index_file_path(other_prefix))
        if np.dtype(other.dtype) != np.dtype(self._dtype):
            raise TypeError("merge_file_: element types differ")
        d0, m0 = self._data_offsets[-1], self._dim_offsets[-1]
        self._data_offsets.extend(int(d0 + v) for v in other.data_offsets[1:])
        self._dim_offsets.extend(int(m0 + v) for v in other.dim_offsets[1:])
        self._dims.extend(int(v) for v in other.sizes)
        self._append_file(other_prefix)

    def finalize(self, index_file: str):
        self._bin.close()
        LegacyIndex(self._dtype, np.dtype(self._dtype).itemsize, np.asarray(self._dim_offsets),
                    np.asarray(self._data_offsets), np.asarray(self._dims), np.asarray(self._doc_idx)).store(index_file)


class MMapIndexedDatasetBuilder(_StreamWriter):
    """Writer of the mmap layout (1-D token sequences)."""

    def __init__(self, out_file: str, dtype=np.int64):
        super().__init__(out_file, dtype)
        self._sizes: List[int] = []

    def add_item(self, arr):
        arr = np.asarray(arr, dtype=self._dtype)
        self._append_bytes(arr)
        self._sizes.append(arr.size)

    def add_items(self, arrays):
        arrays = [np.asarray(a, dtype=self._dtype) for a in arrays]
        if arrays:
            self._append_bytes(np.concatenate(arrays))
            self._sizes.extend(a.size for a in arrays)

    def end_document(self):
        self._doc_idx.append(len(self._sizes))

    def merge_file_(self, other_prefix: str):
        other = MMapIndex.load(index_file_path(other_prefix))
        if np.dtype(other.dtype) != np.dtype(self._dtype):
            raise TypeError("merge_file_: element types differ")
        shift = len(self._sizes)
        self._sizes.extend(int(n) for n in other.sizes)
        self._doc_idx.extend(int(shift + d) for d in other.doc_idx[1:])
        self._append_file(other_prefix)

    def finalize(self, index_file: str):
        self._bin.close()
        MMapIndex.store(index_file, self._dtype, self._sizes, self._doc_idx)


def read_longs(f, n: int):
    """``n`` little-endian int64 values from the binary file object ``f``."""
    a = np.empty(int(n), dtype=np.int64)
    got = f.readinto(a)
    if got != a.nbytes:
        raise EOFError(f"wanted {a.nbytes} bytes, file had {got}")
    return a


def write_longs(f, a):
    """Write the sequence ``a`` to ``f`` as int64."""
    f.write(np.asarray(a, dtype=np.int64).tobytes())
