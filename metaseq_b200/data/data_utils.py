"""Batching helpers.  The inner loops of ``batch_by_size`` run in the host C++ library when
it is built (``csrc/host/batching.cpp``) and in numpy/python otherwise; both produce the same
batches (reference: metaseq/data/data_utils.py:203-257 and data_utils_fast.pyx:20-178)."""
from __future__ import annotations

import contextlib
import ctypes
import itertools
import logging
import os
from typing import List, Optional

import numpy as np
import torch

logger = logging.getLogger(__name__)


def collate_tokens(values, pad_idx, eos_idx=None, left_pad=False, move_eos_to_beginning=False, pad_to_length=None,
                   pad_to_multiple=1, pad_to_bsz=None):
    """1-D tensors -> padded 2-D tensor."""
    size = max(v.size(0) for v in values)
    size = size if pad_to_length is None else max(size, pad_to_length)
    if pad_to_multiple != 1 and size % pad_to_multiple != 0:
        size = int(((size - 0.1) // pad_to_multiple + 1) * pad_to_multiple)
    batch = len(values) if pad_to_bsz is None else max(len(values), pad_to_bsz)
    res = values[0].new(batch, size).fill_(pad_idx)
    for i, v in enumerate(values):
        dst = res[i][size - len(v):] if left_pad else res[i][: len(v)]
        if move_eos_to_beginning:
            if eos_idx is None:
                dst[0] = v[-1]
            else:
                dst[0] = eos_idx
            dst[1:] = v[:-1]
        else:
            dst.copy_(v)
    return res


def _filter_by_size_dynamic(indices, size_fn, max_positions, raise_exception=False):
    def ok(idx):
        s = size_fn(idx)
        if isinstance(max_positions, (float, int)):
            return s <= max_positions
        if isinstance(s, (tuple, list)) and isinstance(max_positions, (tuple, list)):
            return all(a is None or b is None or a <= b for a, b in zip(s, max_positions))
        return all(a <= max_positions[0] for a in (s if isinstance(s, (tuple, list)) else [s]))

    ignored = []
    kept = []
    for i in indices:
        (kept if ok(i) else ignored).append(i)
    return np.asarray(kept, dtype=np.int64), ignored


def batch_fixed(indices, bsz):
    for i in range(0, len(indices), bsz):
        yield list(indices[i:i + bsz])


def _host_lib():
    from metaseq_b200.ops import _lib

    return _lib.host()


def batch_by_size_py(indices, num_tokens_vec, max_tokens, max_sentences, bsz_mult):
    """Greedy batching in index order.  A batch is closed when adding the next sample would
    exceed ``max_sentences`` rows or ``rows * longest > max_tokens``; the closed batch is cut to
    the largest multiple of ``bsz_mult`` (or kept whole when shorter than one multiple) and
    the remainder starts the next batch."""
    batches = []
    batch: List[int] = []
    lens: List[int] = []
    longest = 0
    for k, idx in enumerate(indices):
        n = int(num_tokens_vec[k])
        lens.append(n)
        longest = max(longest, n)
        rows = len(batch)
        full = rows > 0 and ((max_sentences > 0 and rows == max_sentences) or
                             (max_tokens > 0 and (rows + 1) * longest > max_tokens))
        if full:
            cut = max(bsz_mult * (rows // bsz_mult), rows % bsz_mult)
            batches.append(batch[:cut])
            batch = batch[cut:]
            lens = lens[cut:]
            longest = max(lens) if lens else 0
        batch.append(int(idx))
    if batch:
        batches.append(batch)
    return batches


def batch_by_size(indices, num_tokens_fn=None, num_tokens_vec=None, max_tokens=None, max_sentences=None,
                  required_batch_size_multiple=1, fixed_shapes=None):
    max_tokens = int(max_tokens) if max_tokens is not None else -1
    max_sentences = int(max_sentences) if max_sentences is not None else -1
    bsz_mult = int(required_batch_size_multiple)
    if not isinstance(indices, np.ndarray):
        indices = np.fromiter(indices, dtype=np.int64, count=-1)
    indices = indices.astype(np.int64, copy=False)
    if num_tokens_vec is None:
        num_tokens_vec = np.fromiter((num_tokens_fn(int(i)) for i in indices), dtype=np.int64, count=len(indices))
    else:
        num_tokens_vec = np.asarray(num_tokens_vec, dtype=np.int64)
    if fixed_shapes is not None:
        return batch_fixed_shapes(indices, num_tokens_vec, np.asarray(fixed_shapes, dtype=np.int64))
    lib = _host_lib()
    if lib is not None and hasattr(lib, "msq_batch_by_size"):
        n = len(indices)
        ends = np.zeros(n + 1, dtype=np.int64)
        fn = lib.msq_batch_by_size
        fn.restype = ctypes.c_longlong
        nb = fn(num_tokens_vec.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(n), ctypes.c_longlong(max_tokens),
                ctypes.c_longlong(max_sentences), ctypes.c_longlong(bsz_mult), ends.ctypes.data_as(ctypes.c_void_p))
        out, start = [], 0
        for b in range(int(nb)):
            out.append(indices[start:ends[b]].tolist())
            start = int(ends[b])
        return out
    return batch_by_size_py(indices, num_tokens_vec, max_tokens, max_sentences, bsz_mult)


def batch_fixed_shapes_py(indices, num_tokens_vec, fixed_shapes):
    out, batch, longest = [], [], 0
    for k, idx in enumerate(indices):
        n = int(num_tokens_vec[k])
        cand = max(longest, n)
        fits = any(len(batch) + 1 <= r and cand <= t for r, t in fixed_shapes)
        if not fits and batch:
            out.append(batch)
            batch, longest = [], 0
        batch.append(int(idx))
        longest = max(longest, n)
    if batch:
        out.append(batch)
    return out


def batch_fixed_shapes(indices, num_tokens_vec, fixed_shapes):
    """``fixed_shapes``: rows of (batch rows, longest element).  Samples are taken in order; the open batch grows
    while some shape still holds it and is closed by the first sample that fits no shape together with it
    (reference: ``batch_fixed_shapes_fast``, metaseq/data/data_utils_fast.pyx:124-172, which leaves the sample that
    opens a batch out of that batch's longest-element count; here it counts).  Native loop when the host library
    is built."""
    fixed_shapes = np.ascontiguousarray(fixed_shapes, dtype=np.int64).reshape(-1, 2)
    lib = _host_lib()
    if lib is not None and hasattr(lib, "msq_batch_fixed_shapes"):
        n = len(indices)
        num_tokens_vec = np.ascontiguousarray(num_tokens_vec, dtype=np.int64)
        ends = np.zeros(n + 1, dtype=np.int64)
        fn = lib.msq_batch_fixed_shapes
        fn.restype = ctypes.c_longlong
        nb = fn(num_tokens_vec.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(n),
                fixed_shapes.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(len(fixed_shapes)),
                ends.ctypes.data_as(ctypes.c_void_p))
        out, start = [], 0
        for b in range(int(nb)):
            out.append([int(i) for i in indices[start:ends[b]]])
            start = int(ends[b])
        return out
    return batch_fixed_shapes_py(indices, num_tokens_vec, fixed_shapes.tolist())


def batch_by_size_fn(indices, num_tokens_fn, max_tokens=None, max_sentences=None, required_batch_size_multiple=1):
    """The size-callback form (metaseq/data/data_utils_fast.pyx:106-123): sizes are read through ``num_tokens_fn`` once
    into a vector, the batching itself is the native loop."""
    return batch_by_size(indices, num_tokens_fn=num_tokens_fn, max_tokens=max_tokens, max_sentences=max_sentences,
                         required_batch_size_multiple=required_batch_size_multiple)


@contextlib.contextmanager
def numpy_seed(seed, *addl_seeds):
    from metaseq_b200.utils import numpy_seed as _ns

    with _ns(seed, *addl_seeds):
        yield


def load_indexed_dataset(path, dictionary=None, dataset_impl=None, combine=False, default="cached"):
    """Binary corpus at ``path`` (``.bin`` / ``.idx``).  With ``combine`` the numbered continuations
    ``path1, path2, ...`` are concatenated behind it.  ``None`` when nothing exists at ``path``
    (reference: metaseq/data/data_utils.py, ``load_indexed_dataset``)."""
    from metaseq_b200.data import indexed_dataset
    from metaseq_b200.data.concat_dataset import ConcatDataset

    found = []
    k = 0
    while True:
        prefix = path + (str(k) if k > 0 else "")
        impl = dataset_impl or indexed_dataset.infer_dataset_impl(prefix)
        if impl is None or not indexed_dataset.dataset_exists(prefix, impl):
            break
        found.append(indexed_dataset.make_dataset(prefix, impl or default, fix_lua_indexing=True, dictionary=dictionary))
        if not combine:
            break
        k += 1
    if not found:
        return None
    return found[0] if len(found) == 1 else ConcatDataset(found)



def collect_filtered(function, iterable, filtered: list):
    """Like ``filter``, but the rejected elements are appended to ``filtered``."""
    for element in iterable:
        if function(element):
            yield element
        else:
            filtered.append(element)


_JOINERS = {"sentencepiece": "▁", "wordpiece": "_", "letter": "|", "_EOW": "_EOW"}


def post_process(sentence: str, symbol: Optional[str]) -> str:
    """Undoes a sub-word segmentation written with spaces between pieces: the pieces are joined and the scheme's
    word-boundary mark becomes a space (metaseq/data/data_utils.py:260-273)."""
    if symbol is None or symbol == "none":
        return sentence
    if symbol not in _JOINERS:
        raise NotImplementedError(f"Unknown post_process option: {symbol}")
    return sentence.replace(" ", "").replace(_JOINERS[symbol], " ").strip()


def _find_extra_valid_paths(dataset_path: str) -> set:
    """Names (without extension) of the numbered validation sets (``valid1``, ``valid2.bin`` ...) in the local
    directories of ``dataset_path``."""
    import re

    from metaseq_b200 import utils
    from metaseq_b200.file_io import PathManager

    found = set()
    for sub_dir in utils.split_paths(dataset_path):
        if "://" in sub_dir or not os.path.isdir(sub_dir):
            continue
        for entry in PathManager.ls(sub_dir):
            name = os.path.basename(entry.rstrip("/"))
            if re.match(r"valid*[0-9].*", name) is not None:
                found.add(os.path.splitext(name)[0])
    return found


def raise_if_valid_subsets_unintentionally_ignored(train_cfg) -> None:
    """Numbered validation sets on disk that ``--valid-subset`` does not name are an error unless they are combined
    (``--combine-valid-subsets``), deliberately ignored (``--ignore-unused-valid-subsets``) or validation is off
    (metaseq/data/data_utils.py:290-305)."""
    ds = train_cfg.dataset
    data = getattr(train_cfg.task, "data", None)
    if ds.ignore_unused_valid_subsets or ds.combine_valid_subsets or ds.disable_validation or data is None:
        return
    named = ds.valid_subset.split(",")
    ignored = sorted(p for p in _find_extra_valid_paths(data) if p not in named)
    if ignored:
        raise ValueError(f"Valid paths {ignored} will be ignored. Set --combine-val to combine them or "
                         "--ignore-unused-valid-subsets to ignore them.")
