"""Fixed sinusoidal positions (any length); padding positions map to a zero row.  The module can be compiled
with ``torch.jit.script`` (the reference exports it that way: tests/test_export.py:98-103)."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
from torch import Tensor


class SinusoidalPositionalEmbedding(nn.Module):
    """Row ``p`` of the table is ``[sin(p * f_0), ..., sin(p * f_{h-1}), cos(p * f_0), ..., cos(p * f_{h-1})]`` with
    ``h = dim // 2`` and frequencies falling geometrically from 1 to 1/10000 (an odd ``dim`` gets a zero column at
    the end).  Non-padding tokens are numbered from ``padding_idx + 1``; the table grows when a longer input comes."""

    def __init__(self, embedding_dim: int, padding_idx: Optional[int], init_size: int = 1024):
        super().__init__()
        self.embedding_dim = embedding_dim
        self.padding_idx: int = 0 if padding_idx is None else padding_idx
        self.max_positions = int(1e5)
        self.register_buffer("weights", self.get_embedding(init_size, embedding_dim, padding_idx), persistent=False)

    @staticmethod
    def get_embedding(num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None) -> Tensor:
        half = embedding_dim // 2
        decay = math.log(10000.0) / max(1, half - 1)
        freq = torch.exp(-decay * torch.arange(half, dtype=torch.float))
        angle = torch.outer(torch.arange(num_embeddings, dtype=torch.float), freq)
        table = torch.zeros(num_embeddings, embedding_dim)
        table[:, :half] = torch.sin(angle)
        table[:, half:2 * half] = torch.cos(angle)
        if padding_idx is not None:
            table[padding_idx] = 0.0
        return table

    def forward(self, tokens: Tensor, incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]] = None,
                timestep: Optional[Tensor] = None, positions: Optional[Tensor] = None) -> Tensor:
        """``tokens``: ``[batch, length]`` -> ``[batch, length, dim]``.  While decoding step by step
        (``incremental_state`` given) only the newest position is returned, ``[batch, 1, dim]``: ``timestep + 1``
        if a time step is given, else the input length."""
        batch, length = tokens.shape[0], tokens.shape[1]
        needed = self.padding_idx + 1 + length
        if needed > self.weights.size(0):
            self.weights = self.get_embedding(needed, self.embedding_dim, self.padding_idx).to(self.weights)
        if incremental_state is not None:
            newest = length
            if timestep is not None:
                newest = int(timestep.view(-1)[0]) + 1
            return self.weights[self.padding_idx + newest].expand(batch, 1, -1)
        if positions is None:
            # non-padding tokens count from padding_idx + 1 (as utils.make_positions does)
            real = tokens.ne(self.padding_idx).to(torch.int32)
            positions = (torch.cumsum(real, dim=1).to(torch.int32) * real).to(torch.int64) + self.padding_idx
        return self.weights.index_select(0, positions.view(-1)).view(batch, length, -1).detach()
