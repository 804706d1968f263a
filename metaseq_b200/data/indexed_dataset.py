"""On-disk token datasets in the two binary layouts used by fairseq-family tools, plus a raw-text dataset
(reference: metaseq/data/indexed_dataset.py).  The layouts are a compatibility contract:

``mmap``  (``<prefix>.idx`` / ``<prefix>.bin``)
    idx: magic ``MMIDIDX\\0\\0`` | uint64 version (1) | uint8 dtype code | uint64 n |
         int32 sizes[n] | int64 byte pointers[n];   bin: the items back to back.
``lazy`` / ``cached``  (legacy "TNTIDX" layout, token ids stored 1-based)
    idx: magic ``TNTIDX\\0\\0`` | uint64 version (1) | uint64 dtype code | uint64 element size |
         uint64 n | uint64 s | int64 dim_offsets[n+1] | int64 data_offsets[n+1] | int64 sizes[s].

Both readers map the ``.bin`` file once (``np.memmap``) and slice it per item; the legacy "cached" variant
additionally materialises the requested items in memory on ``prefetch``.
"""
from __future__ import annotations

import shutil
import struct
from typing import Dict, Optional

import numpy as np
import torch

from metaseq_b200.file_io import PathManager

from .base_dataset import BaseDataset

DTYPE_CODES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}
MMAP_MAGIC = b"MMIDIDX\x00\x00"   # 9 bytes
LEGACY_MAGIC = b"TNTIDX\x00\x00"  # 8 bytes
_U64 = struct.Struct("<Q")
_U8 = struct.Struct("<B")


def index_file_path(prefix_path):
    return prefix_path + ".idx"


def data_file_path(prefix_path):
    return prefix_path + ".bin"


def _pair_exists(prefix) -> bool:
    return all(PathManager.exists(p) for p in (index_file_path(prefix), data_file_path(prefix)))


def _dtype_header_code(dtype) -> int:
    matches = [code for code, dt in DTYPE_CODES.items() if dt == dtype]
    if not matches:
        raise ValueError(dtype)
    return matches[0]


def best_fitting_int_dtype(max_int_to_represent=None):
    """Smallest unsigned type that holds a vocabulary of this size."""
    if max_int_to_represent is None or max_int_to_represent >= 65500:
        return np.int64 if (max_int_to_represent or 0) >= 4294967295 else np.uint32
    return np.uint16


def read_longs(f, n):
    return np.frombuffer(f.read(8 * n), dtype=np.int64).copy()


def write_longs(f, a):
    f.write(np.asarray(a, dtype=np.int64).tobytes())


def get_available_dataset_impl():
    return ["raw", "lazy", "cached", "mmap"]


def infer_dataset_impl(path) -> Optional[str]:
    if PathManager.exists(path) and not PathManager.exists(index_file_path(path)):
        return "raw"
    if not _pair_exists(path):
        return None
    with open(index_file_path(path), "rb") as f:
        head = f.read(9)
    if head == MMAP_MAGIC:
        return "mmap"
    if head[:8] == LEGACY_MAGIC:
        return "cached"
    return None


def dataset_exists(path, impl):
    return PathManager.exists(path) if impl == "raw" else _pair_exists(path)


def make_dataset(path, impl, fix_lua_indexing=False, dictionary=None):
    if not dataset_exists(path, impl):
        return None
    if impl == "raw":
        assert dictionary is not None
        return IndexedRawTextDataset(path, dictionary)
    if impl == "mmap":
        return MMapIndexedDataset(path)
    cls = IndexedCachedDataset if impl == "cached" else IndexedDataset
    return cls(path, fix_lua_indexing=fix_lua_indexing)


def make_builder(out_file, impl, vocab_size=None):
    if impl == "mmap":
        return MMapIndexedDatasetBuilder(out_file, dtype=best_fitting_int_dtype(vocab_size))
    return IndexedDatasetBuilder(out_file)


class _SizedCorpus(BaseDataset):
    """Shared bookkeeping of the binary datasets: ``sizes`` holds the token count of every item."""

    sizes: np.ndarray

    def num_tokens(self, index):
        return self.sizes[index]

    def size(self, index):
        return self.sizes[index]

    def num_tokens_vec(self, indices):
        return np.asarray(self.sizes)[indices]

    @property
    def supports_prefetch(self):
        return False


# ------------------------------------------------------------------ legacy layout
class _LegacyIndex:
    def __init__(self, idx_path):
        with open(idx_path, "rb") as f:
            if f.read(8) != LEGACY_MAGIC:
                raise ValueError("index file does not match the legacy layout; is it an mmap dataset?")
            (version,) = _U64.unpack(f.read(8))
            assert version == 1
            code, self.element_size = struct.unpack("<QQ", f.read(16))
            self.dtype = DTYPE_CODES[code]
            self.n, n_sizes = struct.unpack("<QQ", f.read(16))
            self.dim_offsets = read_longs(f, self.n + 1)
            self.data_offsets = read_longs(f, self.n + 1)
            self.sizes = read_longs(f, n_sizes)


class IndexedDataset(_SizedCorpus):
    """Legacy layout; items are sliced out of a memory map of the data file."""

    def __init__(self, path, fix_lua_indexing=False):
        super().__init__()
        self.path = path
        self.fix_lua_indexing = fix_lua_indexing
        self._data = None
        self.read_index(path)

    def read_index(self, path):
        ix = _LegacyIndex(index_file_path(path))
        self.dtype, self.element_size, self._len = ix.dtype, ix.element_size, ix.n
        self.dim_offsets, self.data_offsets, self.sizes = ix.dim_offsets, ix.data_offsets, ix.sizes

    def read_data(self, path):
        """Maps the data file (done on first access, and again in every worker process)."""
        self._data = np.memmap(data_file_path(path), dtype=self.dtype, mode="r")

    def check_index(self, i):
        if i < 0 or i >= self._len:
            raise IndexError("index out of range")

    def _raw(self, i) -> np.ndarray:
        self.check_index(i)
        if self._data is None:
            self.read_data(self.path)
        shape = tuple(self.sizes[self.dim_offsets[i]:self.dim_offsets[i + 1]])
        return np.asarray(self._data[self.data_offsets[i]:self.data_offsets[i + 1]]).reshape(shape)

    def _finish(self, a: np.ndarray) -> torch.Tensor:
        item = torch.from_numpy(a.astype(np.int64))
        return item - 1 if self.fix_lua_indexing else item

    def __getitem__(self, i) -> torch.Tensor:
        return self._finish(self._raw(i))

    def __len__(self):
        return self._len

    def __getstate__(self):
        state = self.__dict__.copy()
        state["_data"] = None  # workers re-map the file
        return state

    @staticmethod
    def exists(path):
        return _pair_exists(path)


class IndexedCachedDataset(IndexedDataset):
    """Legacy layout with ``prefetch``: the requested items are copied into memory in one pass."""

    def __init__(self, path, fix_lua_indexing=False):
        super().__init__(path, fix_lua_indexing=fix_lua_indexing)
        self._cache: Dict[int, np.ndarray] = {}

    @property
    def supports_prefetch(self):
        return True

    def prefetch(self, indices):
        wanted = sorted(set(int(i) for i in indices) - set(self._cache))
        for i in wanted:
            self._cache[i] = np.array(self._raw(i))
        if wanted:
            self._data = None  # drop the mapping; everything needed is in memory

    def __getitem__(self, i):
        hit = self._cache.get(int(i))
        return self._finish(hit if hit is not None else self._raw(i))


class IndexedDatasetBuilder:
    def __init__(self, out_file, dtype=np.int32):
        self._out = open(out_file, "wb")
        self.dtype = dtype
        self.element_size = np.dtype(dtype).itemsize
        self.data_offsets, self.dim_offsets, self.sizes = [0], [0], []

    def add_item(self, tensor):
        arr = (tensor.numpy() + 1).astype(self.dtype)  # ids are stored 1-based
        self._out.write(arr.tobytes())
        self.data_offsets.append(self.data_offsets[-1] + arr.size)
        self.sizes.extend(tensor.size())
        self.dim_offsets.append(self.dim_offsets[-1] + tensor.dim())

    def merge_file_(self, another_file):
        other = _LegacyIndex(index_file_path(another_file))
        assert other.dtype == self.dtype
        d0, m0 = self.data_offsets[-1], self.dim_offsets[-1]
        self.data_offsets.extend(int(d0 + o) for o in other.data_offsets[1:])
        self.dim_offsets.extend(int(m0 + o) for o in other.dim_offsets[1:])
        self.sizes.extend(int(s) for s in other.sizes)
        with open(data_file_path(another_file), "rb") as src:
            shutil.copyfileobj(src, self._out)

    def finalize(self, index_file):
        self._out.close()
        with open(index_file, "wb") as f:
            f.write(LEGACY_MAGIC)
            f.write(_U64.pack(1))
            f.write(struct.pack("<QQ", _dtype_header_code(self.dtype), self.element_size))
            f.write(struct.pack("<QQ", len(self.data_offsets) - 1, len(self.sizes)))
            for arr in (self.dim_offsets, self.data_offsets, self.sizes):
                write_longs(f, arr)


# -------------------------------------------------------------------- mmap layout
class _MMapIndex:
    def __init__(self, idx_path):
        raw = np.memmap(idx_path, mode="r", dtype=np.uint8)
        if bytes(raw[:9]) != MMAP_MAGIC:
            raise ValueError("index file does not match the mmap layout")
        (version,) = _U64.unpack(bytes(raw[9:17]))
        assert version == 1
        (code,) = _U8.unpack(bytes(raw[17:18]))
        (self.n,) = _U64.unpack(bytes(raw[18:26]))
        self.dtype = DTYPE_CODES[code]
        self._raw = raw
        self.sizes = np.frombuffer(raw, dtype=np.int32, count=self.n, offset=26)
        self.pointers = np.frombuffer(raw, dtype=np.int64, count=self.n, offset=26 + 4 * self.n)

    @staticmethod
    def write(idx_path, dtype, sizes):
        sizes = np.asarray(sizes, dtype=np.int64)
        pointers = np.concatenate([[0], np.cumsum(sizes[:-1] * np.dtype(dtype).itemsize)]).astype(np.int64) \
            if len(sizes) else np.zeros(0, dtype=np.int64)
        with open(idx_path, "wb") as f:
            f.write(MMAP_MAGIC)
            f.write(_U64.pack(1))
            f.write(_U8.pack(_dtype_header_code(dtype)))
            f.write(_U64.pack(len(sizes)))
            f.write(sizes.astype(np.int32).tobytes())
            f.write(pointers.tobytes())


class MMapIndexedDataset(_SizedCorpus):
    def __init__(self, path):
        super().__init__()
        self._open(path)

    def _open(self, path):
        self._path = path
        self._index = _MMapIndex(index_file_path(path))
        self._bin = np.memmap(data_file_path(path), mode="r", dtype=np.uint8)

    def __getstate__(self):
        return self._path

    def __setstate__(self, path):
        self._open(path)

    def __len__(self):
        return self._index.n

    def __getitem__(self, i):
        ptr, n = int(self._index.pointers[i]), int(self._index.sizes[i])
        arr = np.frombuffer(self._bin, dtype=self._index.dtype, count=n, offset=ptr)
        return torch.from_numpy(arr.astype(np.int64))

    @property
    def sizes(self):
        return self._index.sizes

    @staticmethod
    def exists(path):
        return _pair_exists(path)


class MMapIndexedDatasetBuilder:
    def __init__(self, out_file, dtype=np.int64):
        self._out = open(out_file, "wb")
        self._dtype = dtype
        self._sizes = []

    def add_item(self, tensor):
        arr = tensor.numpy().astype(self._dtype)
        self._out.write(arr.tobytes(order="C"))
        self._sizes.append(arr.size)

    def merge_file_(self, another_file):
        other = _MMapIndex(index_file_path(another_file))
        assert other.dtype == self._dtype
        self._sizes.extend(int(s) for s in other.sizes)
        with open(data_file_path(another_file), "rb") as src:
            shutil.copyfileobj(src, self._out)

    def finalize(self, index_file):
        self._out.close()
        _MMapIndex.write(index_file, self._dtype, self._sizes)


def get_indexed_dataset_to_local(path) -> str:
    """Fetches ``<path>.idx`` / ``<path>.bin`` through the path manager and returns the local prefix."""
    local_idx = PathManager.get_local_path(index_file_path(path))
    local_bin = PathManager.get_local_path(data_file_path(path))
    prefix = local_bin[: -len(".bin")]
    assert local_idx == prefix + ".idx", (local_idx, local_bin)
    return prefix


# ---------------------------------------------------------------------- raw text
class IndexedRawTextDataset(_SizedCorpus):
    """One sentence per line of a text file, tokenised with the dictionary at load time."""

    def __init__(self, path, dictionary, append_eos=True, reverse_order=False):
        super().__init__()
        self.append_eos, self.reverse_order = append_eos, reverse_order
        self.read_data(path, dictionary)

    def read_data(self, path, dictionary):
        with open(path, "r", encoding="utf-8") as f:
            self.lines = [ln.rstrip("\n") for ln in f]
        self.tokens_list = [dictionary.encode_line(ln, add_if_not_exist=False, append_eos=self.append_eos,
                                                   reverse_order=self.reverse_order).long() for ln in self.lines]
        self.sizes = np.array([len(t) for t in self.tokens_list])

    def check_index(self, i):
        if i < 0 or i >= len(self.tokens_list):
            raise IndexError("index out of range")

    def __getitem__(self, i):
        self.check_index(i)
        return self.tokens_list[i]

    def get_original_text(self, i):
        self.check_index(i)
        return self.lines[i]

    def __len__(self):
        return len(self.tokens_list)

    @staticmethod
    def exists(path):
        return PathManager.exists(path)
