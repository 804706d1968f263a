"""Evaluation wrapper that carries the last ``context_window`` tokens of the corpus forward: each sample is
prefixed with them so early positions are scored with context, and ``start_indices`` tells the scorer where the
new tokens begin (reference: metaseq/data/lm_context_window_dataset.py:15-97)."""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from .base_wrapper_dataset import BaseWrapperDataset


class LMContextWindowDataset(BaseWrapperDataset):
    def __init__(self, dataset, tokens_per_sample: int, context_window: int, pad_idx: int):
        super().__init__(dataset)
        assert context_window > 0
        self.tokens_per_sample = tokens_per_sample
        self.context_window = context_window
        self.pad_idx = pad_idx
        self.prev_tokens = torch.empty(0, dtype=torch.long)  # running tail of the corpus seen so far

    def collater(self, samples) -> Dict:
        batch = self.dataset.collater(samples)
        src, tgt = batch["net_input"]["src_tokens"], batch["target"]
        lengths = batch["net_input"]["src_lengths"]
        bsz, width = src.shape
        limit = self.tokens_per_sample + self.context_window
        out_src = src.new_full((bsz, width + self.context_window), self.pad_idx)
        out_tgt = tgt.new_full((bsz, width + self.context_window), self.pad_idx)
        starts = []
        for row in range(bsz):
            n_real = int(src[row].ne(self.pad_idx).sum())
            overflow = self.prev_tokens.numel() + n_real - limit
            if overflow > 0:
                self.prev_tokens = self.prev_tokens[overflow:]
            ctx = self.prev_tokens.numel()
            out_src[row, :ctx] = self.prev_tokens
            out_src[row, ctx:ctx + width] = src[row]
            out_tgt[row, ctx:ctx + tgt.shape[1]] = tgt[row]
            starts.append(ctx)
            lengths[row] += ctx
            real = out_src[row][out_src[row] != self.pad_idx]
            self.prev_tokens = real[-self.context_window:].clone()
        batch["net_input"]["src_tokens"] = out_src
        batch["target"] = out_tgt
        batch["start_indices"] = starts
        return batch

    def ordered_indices(self):
        # the carried context only makes sense in corpus order
        return np.arange(len(self.dataset))
