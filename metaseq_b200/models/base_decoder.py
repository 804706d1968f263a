"""Decoder base classes (reference: metaseq/models/base_decoder.py)."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from metaseq_b200 import utils


class BaseDecoder(nn.Module):
    def __init__(self, dictionary):
        super().__init__()
        self.dictionary = dictionary

    def forward(self, prev_output_tokens, **kwargs):
        x, extra = self.extract_features(prev_output_tokens, **kwargs)
        return self.output_layer(x), extra

    def extract_features(self, prev_output_tokens, **kwargs):
        raise NotImplementedError

    def output_layer(self, features, **kwargs):
        raise NotImplementedError

    def get_normalized_probs(self, logits: torch.Tensor, log_probs: bool, sample=None):
        """fp32 (log-)softmax over the vocabulary."""
        if log_probs:
            return utils.log_softmax(logits, dim=-1)
        return utils.softmax(logits, dim=-1)

    def reorder_incremental_state(self, incremental_state, new_order):
        """Called when the batch order changes between decoding steps (beam search); nothing to do for a decoder
        without per-step state."""
        pass

    def max_positions(self):
        return 1e6


class IncrementalDecoder(BaseDecoder):
    """Decoder that can consume one step at a time, keeping per-layer state in ``incremental_state``."""

    def reorder_incremental_state(self, incremental_state, new_order):
        for m in self.modules():
            if m is not self and hasattr(m, "reorder_incremental_state"):
                m.reorder_incremental_state(incremental_state, new_order)
