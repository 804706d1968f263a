"""Fixed sinusoidal positions (any length); padding positions map to a zero row.  The module can be compiled
with ``torch.jit.script`` (the reference exports it that way: tests/test_export.py:98-103)."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
from torch import Tensor


class SinusoidalPositionalEmbedding(nn.Module):
    def __init__(self, embedding_dim: int, padding_idx: Optional[int], init_size: int = 1024):
        super().__init__()
        self.embedding_dim = embedding_dim
        self.padding_idx: int = padding_idx if padding_idx is not None else 0
        self.register_buffer("weights", self.get_embedding(init_size, embedding_dim, padding_idx), persistent=False)
        self.max_positions = int(1e5)

    @staticmethod
    def get_embedding(num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None) -> Tensor:
        half = embedding_dim // 2
        freq = torch.exp(torch.arange(half, dtype=torch.float) * -(math.log(10000.0) / max(1, half - 1)))
        ang = torch.arange(num_embeddings, dtype=torch.float).unsqueeze(1) * freq.unsqueeze(0)
        emb = torch.cat([torch.sin(ang), torch.cos(ang)], dim=1).view(num_embeddings, -1)
        if embedding_dim % 2 == 1:
            emb = torch.cat([emb, torch.zeros(num_embeddings, 1)], dim=1)
        if padding_idx is not None:
            emb[padding_idx, :] = 0
        return emb

    def forward(self, tokens: Tensor, incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]] = None,
                timestep: Optional[Tensor] = None, positions: Optional[Tensor] = None) -> Tensor:
        bsz, seq_len = tokens.shape[0], tokens.shape[1]
        max_pos = self.padding_idx + 1 + seq_len
        if max_pos > self.weights.size(0):
            self.weights = self.get_embedding(max_pos, self.embedding_dim, self.padding_idx).to(self.weights)
        if positions is None:
            # non-padding tokens count from padding_idx + 1 (as utils.make_positions does)
            mask = tokens.ne(self.padding_idx).to(torch.int32)
            positions = (torch.cumsum(mask, dim=1).to(torch.int32) * mask).to(torch.int64) + self.padding_idx
        return self.weights.index_select(0, positions.view(-1)).view(bsz, seq_len, -1).detach()
