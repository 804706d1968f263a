"""Map-style dataset that cuts a corpus of variable-length items into blocks of tokens
(reference: metaseq/data/token_block_dataset.py:15-206).  The slicing and the block -> item index run in
the native host library (``csrc/host/batching.cpp``), with a Python restatement as fallback."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import data_utils
from .base_dataset import BaseDataset

_MODES = {"none": 0, None: 0, "complete": 1, "complete_doc": 2, "eos": 3}


def get_slice_indices(sizes: np.ndarray, break_mode, block_size: int, document_sep_len: int = 1) -> np.ndarray:
    sizes = np.ascontiguousarray(sizes, dtype=np.int64)
    mode = _MODES[break_mode]
    lib = data_utils._host_lib()
    if lib is not None:
        cap = 2 * (len(sizes) + int(sizes.sum()) // max(1, block_size) + 2)
        out = np.empty((cap, 2), dtype=np.int64)
        nb = lib.msq_token_block_slices(sizes.ctypes.data_as(ctypes.c_void_p), len(sizes), int(block_size), mode,
                                        int(document_sep_len), out.ctypes.data_as(ctypes.c_void_p))
        return out[:nb].copy()
    return get_slice_indices_py(sizes, break_mode, block_size, document_sep_len)


def get_slice_indices_py(sizes, break_mode, block_size, document_sep_len=1) -> np.ndarray:
    mode = _MODES[break_mode]
    out = []
    if mode == 0:
        total = int(np.sum(sizes))
        for s in range(0, total, block_size):
            out.append((s, min(s + block_size, total)))
    elif mode in (1, 2):
        tok, cur = 0, 0
        for sz in sizes:
            sz = int(sz)
            if mode == 2 and sz == document_sep_len:  # document separator: close the block
                if cur > 0:
                    out.append((tok, tok + cur))
                tok += cur + sz
                cur = 0
                continue
            if cur + sz <= block_size or cur == 0:
                cur += sz
            else:
                out.append((tok, tok + cur))
                tok += cur
                cur = sz
        if cur > 0:
            out.append((tok, tok + cur))
    else:  # eos: one item per block
        tok = 0
        for sz in sizes:
            out.append((tok, tok + int(sz)))
            tok += int(sz)
    return np.asarray(out, dtype=np.int64).reshape(-1, 2)


def get_block_to_dataset_index(sizes: np.ndarray, slices: np.ndarray) -> np.ndarray:
    sizes = np.ascontiguousarray(sizes, dtype=np.int64)
    slices = np.ascontiguousarray(slices, dtype=np.int64)
    lib = data_utils._host_lib()
    out = np.empty((len(slices), 3), dtype=np.int64)
    if lib is not None and len(slices):
        lib.msq_block_to_dataset_index(sizes.ctypes.data_as(ctypes.c_void_p), len(sizes),
                                       slices.ctypes.data_as(ctypes.c_void_p), len(slices),
                                       out.ctypes.data_as(ctypes.c_void_p))
        return out
    cum = np.concatenate([[0], np.cumsum(sizes)])
    for b, (s, e) in enumerate(slices):
        first = int(np.searchsorted(cum, s, side="right") - 1)
        last = int(np.searchsorted(cum, e - 1, side="right") - 1) if e > s else first
        out[b] = (first, s - cum[first], last)
    return out


class TokenBlockDataset(BaseDataset):
    """``break_mode``: ``none`` (blocks may cross items), ``complete`` (whole items up to ``block_size``),
    ``complete_doc`` (as complete, never crossing an empty-line document separator), ``eos`` (one item per
    block).  ``include_targets`` yields ``(source, future_target, past_target)`` for language modeling."""

    def __init__(self, dataset, sizes, block_size, pad, eos, break_mode=None, include_targets=False,
                 document_sep_len=1, use_plasma_view=False, split_path=None, plasma_path=None):
        super().__init__()
        self.dataset = dataset
        self.pad = pad
        self.eos = eos
        self.include_targets = include_targets
        assert len(dataset) > 0
        assert len(dataset) == len(sizes)
        sizes = np.asarray(sizes, dtype=np.int64)
        self._slice_indices = get_slice_indices(sizes, break_mode if break_mode is not None else "none", block_size,
                                                document_sep_len)
        self._sizes = self._slice_indices[:, 1] - self._slice_indices[:, 0]
        if break_mode == "eos":
            n = len(sizes)
            self._block_to_dataset_index = np.stack([np.arange(n), np.zeros(n, dtype=np.int64), np.arange(n)], 1)
        else:
            self._block_to_dataset_index = get_block_to_dataset_index(sizes, self._slice_indices)

    @property
    def slice_indices(self):
        return self._slice_indices

    @property
    def sizes(self):
        return self._sizes

    @property
    def block_to_dataset_index(self):
        return self._block_to_dataset_index

    def attr(self, attr: str, index: int):
        start_ds_idx, _, _ = self.block_to_dataset_index[index]
        return self.dataset.attr(attr, start_ds_idx)

    def __getitem__(self, index):
        start_ds_idx, start_offset, end_ds_idx = (int(x) for x in self.block_to_dataset_index[index])
        buffer = torch.cat([self.dataset[idx] for idx in range(start_ds_idx, end_ds_idx + 1)])
        s, e = (int(x) for x in self.slice_indices[index])
        length = e - s
        s, e = start_offset, start_offset + length
        item = buffer[s:e]
        if not self.include_targets:
            return item
        # source is shifted right by one (wrapping to eos at the very start), past target by two
        if s == 0:
            source = torch.cat([item.new([self.eos]), buffer[0:e - 1]])
            past_target = torch.cat([item.new([self.pad, self.eos]), buffer[0:e - 2]])
        else:
            source = buffer[s - 1:e - 1]
            if s == 1:
                past_target = torch.cat([item.new([self.eos]), buffer[0:e - 2]])
            else:
                past_target = buffer[s - 2:e - 2]
        return source, item, past_target

    def __len__(self):
        return len(self.slice_indices)

    def num_tokens(self, index):
        return int(self._sizes[index])

    def num_tokens_vec(self, indices):
        return self._sizes[indices]

    def size(self, index):
        return int(self._sizes[index])

    @property
    def supports_prefetch(self):
        return getattr(self.dataset, "supports_prefetch", False)

    def prefetch(self, indices):
        self.dataset.prefetch({
            ds_idx
            for index in indices
            for start, _, end in [self.block_to_dataset_index[index]]
            for ds_idx in range(int(start), int(end) + 1)
        })
