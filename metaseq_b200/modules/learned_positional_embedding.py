"""Learned absolute positions.  The table has ``max_positions + padding_idx + 1`` rows and a
token's row is its 1-based count among non-pad tokens plus ``padding_idx`` (so with OPT's
padding_idx = 1 the first token uses row 2).  Reference:
metaseq/modules/learned_positional_embedding.py:23-54, positional_embedding.py:34-47."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from metaseq_b200 import utils


class LearnedPositionalEmbedding(nn.Embedding):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int], **kw):
        super().__init__(num_embeddings, embedding_dim, padding_idx, **kw)
        if self.padding_idx is not None:
            self.max_positions = self.num_embeddings - self.padding_idx - 1
        else:
            self.max_positions = self.num_embeddings

    def positions_for(self, tokens, incremental_state=None, positions=None):
        assert positions is None or self.padding_idx is None, \
            "If positions is pre-computed then padding_idx should not be set."
        if positions is not None:
            return positions
        if incremental_state is not None and tokens.size(1) >= 1 and incremental_state.get("_full_prefix", True):
            # positions depend on the number of non-pad tokens seen so far; callers pass the full prefix
            return utils.make_positions(tokens, self.padding_idx)
        return utils.make_positions(tokens, self.padding_idx)

    def forward(self, tokens, incremental_state=None, positions=None):
        positions = self.positions_for(tokens, incremental_state, positions)
        return TF.embedding(positions, self.weight, self.padding_idx, self.max_norm, self.norm_type,
                            self.scale_grad_by_freq, self.sparse)


def PositionalEmbedding(num_embeddings: int, embedding_dim: int, padding_idx: Optional[int], learned: bool = False,
                        learned_sinusoidal: bool = False, full_megatron_init: bool = False,
                        pos_init_scalar: float = 1.0, megatron_init_sigma=None, truncate_init: bool = False,
                        dtype=None, device=None):
    """Builds the position table with the reference's sizing rule: ``padding_idx + 1`` extra
    rows are added so that position indices starting at ``padding_idx + 1`` fit."""
    if learned or learned_sinusoidal:
        if padding_idx is not None:
            num_embeddings = num_embeddings + padding_idx + 1
        m = LearnedPositionalEmbedding(num_embeddings, embedding_dim, padding_idx, dtype=dtype, device=device)
        with torch.no_grad():
            if full_megatron_init:
                nn.init.normal_(m.weight, mean=0, std=megatron_init_sigma * pos_init_scalar)
            else:
                nn.init.normal_(m.weight, mean=0, std=embedding_dim ** -0.5)
            if padding_idx is not None:
                m.weight[padding_idx].zero_()
        return m
    from .sinusoidal_positional_embedding import SinusoidalPositionalEmbedding

    return SinusoidalPositionalEmbedding(embedding_dim, padding_idx,
                                         init_size=num_embeddings + (padding_idx or 0) + 1)
