"""Streams a document dataset as fixed-length token blocks.

Behaviour follows the reference (metaseq/data/document_to_sequence.py):
documents are permuted per (seed, epoch) (:240-250), split contiguously across
DataLoader workers (:265-274), cut into ``block_size`` blocks by one of four
break modes (``none`` / ``complete`` / ``eos_pad_8`` / ``passthrough``,
:418-526), passed through a shuffle buffer driven by a seeded generator whose
draws are taken in batches of 1024 (:94-129, :317-350), and the first
``to_skip`` sequences are dropped on resume without tokenising the documents
they came from, using a shared cache of document lengths (:27-62, :283-309).

The implementation is organised differently: a block is a list of ``_Span``
objects that point at a shared ``_Doc`` holder, so a document skipped during
fast-forward is never loaded, and one that is needed is loaded exactly once.
"""
from __future__ import annotations

import logging
import math
import time
from ctypes import addressof, c_int, memmove, sizeof
from multiprocessing import Array, Lock
from typing import Iterable, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

logger = logging.getLogger(__name__)


class LockingArray:
    """Shared int array (one slot per document, 0 = length unknown) plus one lock per
    worker.  The trainer takes every lock to read a consistent snapshot into a checkpoint
    while worker processes keep filling the cache."""

    def __init__(self, size: int, num_workers: int = 1):
        self.data = Array(c_int, size, lock=False)
        self.set_num_workers(num_workers)

    def set_num_workers(self, num_workers: int):
        self.worker_locks = [Lock() for _ in range(max(1, num_workers))]

    def __len__(self):
        return len(self.data)

    def __getstate__(self) -> bytes:
        for lock in self.worker_locks:
            lock.acquire()
        try:
            return bytes(self.data)
        finally:
            for lock in self.worker_locks:
                lock.release()

    def __setstate__(self, state: bytes):
        n = len(state) // sizeof(c_int)
        self.__init__(n, 1)
        memmove(addressof(self.data), state, len(state))

    def load_bytes(self, state: bytes):
        n = min(len(state), len(self.data) * sizeof(c_int))
        memmove(addressof(self.data), state, n)


class _Doc:
    """Holder for one document: an index into the dataset until somebody needs the tokens."""

    __slots__ = ("index", "value")

    def __init__(self, index: Optional[int], value=None):
        self.index = index
        self.value = value

    def load(self, dataset):
        if self.value is None:
            self.value = dataset[self.index]
        return self.value


PAD = _Doc(None, "padding")


class _Span:
    __slots__ = ("doc", "start", "length")

    def __init__(self, doc: _Doc, start: int, length: int):
        self.doc, self.start, self.length = doc, start, length


class _Block:
    __slots__ = ("spans", "ids")

    def __init__(self):
        self.spans: List[_Span] = []
        self.ids: List[int] = []


def blocked_random(seed: int, normal_size: int):
    """Seeded ``integers(high)`` source.  While callers keep asking for ``high ==
    normal_size`` the numbers come from 1024-wide batches (numpy's per-call overhead is
    large); the first request for a smaller range rewinds the generator to the start of
    the current batch, replays the numbers already handed out and continues unbatched, so
    the stream equals the unbatched one."""
    rng = np.random.default_rng(seed)
    snap = None
    batch = None
    used = 0
    batched = True

    def integers(high: int) -> int:
        nonlocal snap, batch, used, batched
        if batched:
            if high == normal_size:
                pos = used % 1024
                if pos == 0:
                    snap = rng.bit_generator.state
                    batch = rng.integers(normal_size, size=1024)
                used += 1
                return int(batch[pos])
            if snap is not None:
                rng.bit_generator.state = snap
                rng.integers(normal_size, size=used % 1024 if used % 1024 else (1024 if used else 0))
            batched = False
        return int(rng.integers(high))

    return integers


# --------------------------------------------------------------- break modes
def _blocks_none(docs: Iterable[Tuple[int, _Doc, int]], block_size: int, drop_last: bool) -> Iterator[_Block]:
    """Concatenate documents and cut every ``block_size`` tokens; a block may span documents."""
    cur = _Block()
    fill = 0
    for idx, (ln, doc, doc_id) in enumerate(docs):
        cur.ids.append(doc_id)
        off = 0
        while ln - off > 0:
            take = min(block_size - fill, ln - off)
            cur.spans.append(_Span(doc, off, take))
            fill += take
            off += take
            if fill == block_size:
                yield cur
                cur = _Block()
                fill = 0
                if ln - off > 0:
                    cur.ids.append(doc_id)
    if fill > 0 and not drop_last:
        cur.spans.append(_Span(PAD, 0, block_size - fill))
        yield cur


def _blocks_complete(docs, block_size: int, drop_last: bool) -> Iterator[_Block]:
    """Pack whole documents; a block never splits a document unless the document alone is
    longer than the block (then it is truncated to one block)."""
    cur = _Block()
    fill = 0
    for ln, doc, doc_id in docs:
        if ln == 0:
            continue
        if ln > block_size:
            ln = block_size
        if fill + ln > block_size:
            cur.spans.append(_Span(PAD, 0, block_size - fill))
            yield cur
            cur = _Block()
            fill = 0
        cur.spans.append(_Span(doc, 0, ln))
        cur.ids.append(doc_id)
        fill += ln
    if fill > 0 and not drop_last:
        cur.spans.append(_Span(PAD, 0, block_size - fill))
        yield cur


def _blocks_eos_pad_8(docs, block_size: int, drop_last: bool) -> Iterator[_Block]:
    """One document per sequence, padded to a multiple of 8, long documents cut at block_size."""
    for ln, doc, doc_id in docs:
        if ln == 0:
            continue
        off = 0
        while off < ln:
            take = min(block_size, ln - off)
            b = _Block()
            b.ids.append(doc_id)
            b.spans.append(_Span(doc, off, take))
            padded = min(block_size, int(math.ceil(take / 8) * 8))
            if padded > take:
                b.spans.append(_Span(PAD, 0, padded - take))
            off += take
            yield b


def _blocks_passthrough(docs, block_size: int, drop_last: bool) -> Iterator[_Block]:
    for ln, doc, doc_id in docs:
        b = _Block()
        b.ids.append(doc_id)
        b.spans.append(_Span(doc, 0, ln))
        yield b


_BREAK_MODES = {
    "none": _blocks_none,
    "complete": _blocks_complete,
    "eos_pad_8": _blocks_eos_pad_8,
    "passthrough": _blocks_passthrough,
}


class DocumentToSequenceDataset(torch.utils.data.IterableDataset):
    """Iterable of ``{"ids": LongTensor[doc indices], "block": LongTensor[tokens]}``.

    Args:
        dataset: map-style dataset of 1-D token tensors (or ``(src, tgt)`` tuples with
            ``source_target=True``).
        block_size: tokens per sequence.
        break_mode: ``none`` | ``complete`` | ``eos_pad_8`` | ``passthrough``.
        drop_last: drop the final partial block instead of padding it.
        padding_idx: fill value of padded positions.
        shuffle_buffer_size: sequences held in the shuffle buffer (1 = no shuffling).
        seed: seed for the document permutation and the shuffle buffer.
        len_cache: optional shared ``LockingArray`` with known document lengths.
        to_skip: sequences to drop at the start (int, or one int per worker).
        permute_documents: shuffle document order each epoch.
        source_target: documents are ``(source, target)`` pairs (fine-tuning).
    """

    def __init__(self, dataset, block_size: int, break_mode: str = "none", drop_last: bool = True,
                 padding_idx: Optional[int] = None, shuffle_buffer_size: int = 1, seed: Optional[int] = None,
                 len_cache: Optional[LockingArray] = None, to_skip: Union[int, Sequence[int]] = 0,
                 permute_documents: bool = True, source_target: bool = False):
        super().__init__()
        if break_mode in (None, ""):
            break_mode = "none"
        if break_mode not in _BREAK_MODES:
            raise ValueError(f"Invalid value for break_mode = {break_mode}. Available options are "
                             f"{sorted(_BREAK_MODES)}.")
        if source_target and break_mode not in ("complete", "eos_pad_8", "passthrough"):
            raise ValueError("source_target documents need break_mode complete, eos_pad_8 or passthrough")
        self.dataset = dataset
        self.block_size = block_size
        self.break_mode = break_mode
        self.drop_last = drop_last
        self.padding_idx = padding_idx
        self.shuffle_buffer_size = max(1, int(shuffle_buffer_size))
        self.to_skip = to_skip
        self.permute_documents = permute_documents
        self.source_target = source_target
        self.worker_offset = 0
        self.document_shuffle_seed = seed
        self.shuffle_buffer_seed = None if seed is None else seed + 2273 + 1284
        self.len_cache = len_cache if len_cache is not None else LockingArray(len(dataset), 1)
        self.indices = None
        self._iterating = False
        self.epoch = None

    def set_epoch(self, epoch: int):
        if hasattr(self.dataset, "set_epoch"):
            self.dataset.set_epoch(epoch)
        self.epoch = epoch
        if self.permute_documents:
            from metaseq_b200.utils import numpy_seed

            with numpy_seed(self.document_shuffle_seed, epoch):
                self.indices = np.random.permutation(len(self.dataset))
        else:
            self.indices = np.arange(len(self.dataset))

    def set_shuffle_buffer_size(self, n: int):
        assert not self._iterating
        self.shuffle_buffer_size = max(1, int(n))

    def set_num_workers(self, num_workers: int):
        self.len_cache.set_num_workers(num_workers)

    # ------------------------------------------------------------------ iteration
    def _documents(self, indices) -> Iterator[Tuple[int, _Doc, int]]:
        cache = self.len_cache.data
        for idx in indices:
            idx = int(idx)
            ln = cache[idx]
            if ln == 0:
                value = self.dataset[idx]
                ln = int(value[0].shape[0] if self.source_target else value.shape[0])
                cache[idx] = ln
                yield ln, _Doc(idx, value), idx
            else:
                yield int(ln), _Doc(idx), idx

    def _shuffled(self, blocks: Iterator[_Block]) -> Iterator[_Block]:
        size = self.shuffle_buffer_size
        draw = blocked_random(self.shuffle_buffer_seed, size) if self.shuffle_buffer_seed is not None \
            else (lambda high: 0)
        buf: List[_Block] = []
        for blk in blocks:
            if len(buf) < size:
                buf.append(blk)
                continue
            j = draw(len(buf))
            out, buf[j] = buf[j], blk
            yield out
        while buf:
            yield buf.pop(draw(len(buf)))

    def _materialise(self, blk: _Block, skip_time: float) -> dict:
        parts = []
        for sp in blk.spans:
            if sp.doc is PAD:
                proto = parts[-1][0] if self.source_target else parts[-1]
                pad = proto.new_full((sp.length,), self.padding_idx)
                parts.append((pad, pad) if self.source_target else pad)
            else:
                value = sp.doc.load(self.dataset)
                if self.source_target:
                    parts.append(tuple(v[sp.start:sp.start + sp.length] for v in value))
                else:
                    parts.append(value[sp.start:sp.start + sp.length])
        out = {"ids": torch.LongTensor(blk.ids), "skip_time": skip_time}
        if self.source_target:
            out["src_block"] = torch.cat([p[0] for p in parts])
            out["tgt_block"] = torch.cat([p[1] for p in parts])
        else:
            out["block"] = torch.cat(parts)
        return out

    def __iter__(self):
        assert not self._iterating, "a DocumentToSequenceDataset can be iterated once per epoch"
        self._iterating = True
        if self.indices is None:
            self.set_epoch(1 if self.epoch is None else self.epoch)
        t0 = time.time()
        info = torch.utils.data.get_worker_info()
        if info is not None and info.num_workers > 1:
            worker = (info.id + self.worker_offset) % info.num_workers
            indices = np.array_split(self.indices, info.num_workers)[worker]
        else:
            worker, indices = 0, self.indices
        to_skip = self.to_skip if isinstance(self.to_skip, int) else self.to_skip[worker]
        lock = self.len_cache.worker_locks[worker % len(self.len_cache.worker_locks)]
        seqs = self._shuffled(_BREAK_MODES[self.break_mode](self._documents(indices), self.block_size, self.drop_last))
        try:
            if to_skip > 0 and worker == 0:
                logger.info(f"Skipping {to_skip} sequences")
            with lock:
                for _ in range(to_skip):
                    next(seqs)
            skip_time = time.time() - t0
            while True:
                with lock:
                    blk = next(seqs)
                yield self._materialise(blk, skip_time)
        except StopIteration:
            return
        finally:
            self._iterating = False
