"""The first-generation streaming datasets: an iterable of documents is cut into fixed-size blocks on the fly
and passed through a shuffle buffer.  Kept for data pipelines written against them; new code uses
``DocumentToSequenceDataset`` (reference: metaseq/data/streaming_token_block_dataset.py,
metaseq/data/streaming_src_tgt_dataset.py).

Items are ``{"ids": LongTensor, "block": LongTensor}`` (token stream) or
``{"ids": ..., "src_block": ..., "tgt_block": ...}`` (source / target pairs, loss only on the target part)."""
from __future__ import annotations

import math
from typing import Callable, Iterable, Optional

import numpy as np
import torch

_PAD_MULTIPLE = 8


def _round_up(n: int, m: int) -> int:
    return int(math.ceil(n / m) * m)


# ----------------------------------------------------------------- block builders (token streams)
def yield_token_blocks(iterable, block_size, drop_last, padding_idx):
    """break mode ``none``: the concatenated stream is cut every ``block_size`` tokens; the tail is padded."""
    pending, ids, have = [], [], 0
    for idx, item in enumerate(iterable):
        ids.append(idx)
        pending.append(item)
        have += item.numel()
        while have >= block_size:
            flat = torch.cat(pending)
            yield {"ids": torch.LongTensor(ids), "block": flat[:block_size]}
            rest = flat[block_size:]
            have = rest.numel()
            pending = [rest] if have else []
            ids = [idx] if have else []
    if have and not drop_last:
        flat = torch.cat(pending)
        pad = flat.new_full((block_size - flat.numel(),), padding_idx)
        yield {"ids": torch.LongTensor(ids), "block": torch.cat([flat, pad])}


def yield_doc_blocks(iterable, block_size, drop_last, padding_idx):
    """break mode ``complete``: blocks hold whole documents (a document longer than a block is cut); each block is
    padded to ``block_size``."""
    cur, ids, used = [], [], 0

    def flush():
        flat = torch.cat(cur)
        pad = flat.new_full((block_size - flat.numel(),), padding_idx)
        return {"ids": torch.LongTensor(ids), "block": torch.cat([flat, pad])}

    for idx, item in enumerate(iterable):
        for start in range(0, item.numel(), block_size):
            piece = item[start:start + block_size]
            if used + piece.numel() > block_size and cur:
                yield flush()
                cur, ids, used = [], [], 0
            cur.append(piece)
            ids.append(idx)
            used += piece.numel()
    if cur and not drop_last:
        yield flush()


def yield_single_sentences_pad_8(iterable, block_size, drop_last, padding_idx):
    """break mode ``eos_pad_8``: one document per block, truncated to ``block_size`` and padded to a multiple of 8."""
    for idx, item in enumerate(iterable):
        item = item[:block_size]
        target = min(block_size, _round_up(item.numel(), _PAD_MULTIPLE))
        pad = item.new_full((target - item.numel(),), padding_idx)
        yield {"ids": torch.LongTensor([idx]), "block": torch.cat([item, pad])}


# -------------------------------------------------------- block builders (source / target pairs)
def _mask_source(src, tgt, padding_idx):
    """Model input is ``src + tgt`` shifted; targets carry padding over the source part."""
    full = torch.cat([src, tgt])
    labels = torch.cat([src.new_full((max(src.numel() - 1, 0),), padding_idx), tgt])
    return full[:-1], labels[: full.numel() - 1] if labels.numel() >= full.numel() - 1 else labels


def yield_src_tgt_blocks(iterable, block_size, drop_last, padding_idx):
    """Packs whole (source, target) pairs into blocks of ``block_size`` positions."""
    srcs, tgts, ids, used = [], [], [], 0

    def flush():
        s, t = torch.cat(srcs), torch.cat(tgts)
        n = block_size - s.numel()
        return {"ids": torch.LongTensor(ids), "src_block": torch.cat([s, s.new_full((n,), padding_idx)]),
                "tgt_block": torch.cat([t, t.new_full((n,), padding_idx)])}

    for idx, (src, tgt) in enumerate(iterable):
        inp, lab = _mask_source(src, tgt, padding_idx)
        inp, lab = inp[:block_size], lab[:block_size]
        if used + inp.numel() > block_size and srcs:
            yield flush()
            srcs, tgts, ids, used = [], [], [], 0
        srcs.append(inp)
        tgts.append(lab)
        ids.append(idx)
        used += inp.numel()
    if srcs and not drop_last:
        yield flush()


def yield_src_tgt_single_sentences_pad_8(iterable, block_size, drop_last, padding_idx):
    for idx, (src, tgt) in enumerate(iterable):
        inp, lab = _mask_source(src, tgt, padding_idx)
        inp, lab = inp[:block_size], lab[:block_size]
        target = min(block_size, _round_up(inp.numel(), _PAD_MULTIPLE))
        n = target - inp.numel()
        yield {"ids": torch.LongTensor([idx]), "src_block": torch.cat([inp, inp.new_full((n,), padding_idx)]),
               "tgt_block": torch.cat([lab, lab.new_full((n,), padding_idx)])}


# ------------------------------------------------------------------------------ datasets
class _StreamingBlocks(torch.utils.data.IterableDataset):
    _BUILDERS: dict = {}

    def __init__(self, dataset: torch.utils.data.IterableDataset, block_size: int, break_mode: str = "none",
                 drop_last: Optional[bool] = False, padding_idx: Optional[int] = None, shuffle_buffer_size: int = 1,
                 seed: Optional[int] = None):
        super().__init__()
        if break_mode in (None, ""):
            break_mode = "none"
        if break_mode not in self._BUILDERS:
            raise ValueError(f'Invalid value for break_mode = {break_mode}. Available options are {sorted(self._BUILDERS)}.')
        if shuffle_buffer_size > 1:
            assert seed is not None, "a shuffle buffer needs a seed"
        self.dataset = dataset
        self.block_size = block_size
        self.break_mode = break_mode
        self.drop_last = drop_last
        self.padding_idx = padding_idx
        self.shuffle_buffer_size = shuffle_buffer_size
        self.seed = seed
        self.block_iterator: Callable = self._BUILDERS[break_mode]
        self.epoch = None

    def set_epoch(self, epoch):
        self.epoch = epoch
        if hasattr(self.dataset, "set_epoch"):
            self.dataset.set_epoch(epoch)

    def set_shuffle_buffer_size(self, new_shuffle_buffer_size):
        assert not self.shuffle_buffer_size > 1 or self.seed is not None
        self.shuffle_buffer_size = new_shuffle_buffer_size

    def __iter__(self) -> Iterable:
        blocks = self.block_iterator(self.dataset, self.block_size, self.drop_last, self.padding_idx)
        if self.shuffle_buffer_size <= 1:
            yield from blocks
            return
        assert self.epoch is not None, "call set_epoch before iterating with a shuffle buffer"
        rng = np.random.default_rng(2273 + self.seed + self.epoch)
        held = []
        for block in blocks:
            if len(held) < self.shuffle_buffer_size:
                held.append(block)
                continue
            j = int(rng.integers(len(held)))
            held[j], block = block, held[j]
            yield block
        while held:
            yield held.pop(int(rng.integers(len(held))))


class StreamingTokenBlockDataset(_StreamingBlocks):
    """Documents (1-D token tensors) -> fixed-size blocks.  ``break_mode``: none | complete | eos_pad_8."""

    _BUILDERS = {"none": yield_token_blocks, "complete": yield_doc_blocks, "eos_pad_8": yield_single_sentences_pad_8}


class StreamingSrcTgtDataset(_StreamingBlocks):
    """(source, target) documents -> blocks with the loss restricted to target positions.
    ``break_mode``: complete | eos_pad_8."""

    _BUILDERS = {"complete": yield_src_tgt_blocks, "eos_pad_8": yield_src_tgt_single_sentences_pad_8}
