"""Structured description of what a self-attention call may look at, beyond plain causality.

The reference hands its attention a dense additive ``[B, T, T]`` (document separator,
metaseq/modules/multihead_attention.py:400-409) or ``[H, T, T]`` (ALiBi,
metaseq/models/transformer_decoder.py:193-230, :474-476) mask.  Here the two cases travel as what they are made
from (one integer per token, one slope per head), which the flash-attention kernels take directly; ``dense``
rebuilds the additive mask for the PyTorch paths (CPU, incremental decoding, padding masks).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch


def alibi_slopes(n_heads: int) -> List[float]:
    """Per-head slopes of "Train Short, Test Long": a geometric sequence for a power-of-two head count, and for other
    counts the sequence of the next lower power of two followed by every second slope of the next higher one."""

    def pow2(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start ** (i + 1) for i in range(n)]

    if math.log2(n_heads).is_integer():
        return pow2(n_heads)
    lower = 2 ** math.floor(math.log2(n_heads))
    return pow2(lower) + alibi_slopes(2 * lower)[0::2][: n_heads - lower]


@dataclass
class AttentionBias:
    """``doc_start``: ``[B, T]`` index of the first token of each token's document (queries see keys from there up to
    themselves).  ``slopes``: ``[H_local]`` fp32; key position times slope is added to the scaled scores."""

    doc_start: Optional[torch.Tensor] = None
    slopes: Optional[torch.Tensor] = None

    def dense(self, T: int, S: int, past: int, device) -> torch.Tensor:
        """Additive fp32 mask ``[B or 1, H or 1, T, S]`` for queries at positions ``past .. past + T - 1`` over keys
        ``0 .. S - 1``, causality included."""
        qpos = torch.arange(past, past + T, device=device).view(1, 1, T, 1)
        kpos = torch.arange(S, device=device).view(1, 1, 1, S)
        banned = kpos > qpos
        if self.doc_start is not None:
            start = self.doc_start.to(device).long()[:, past:past + T].view(-1, 1, T, 1)
            banned = banned | (kpos < start)
        mask = torch.zeros(banned.shape, dtype=torch.float32, device=device).masked_fill_(banned, float("-inf"))
        if self.slopes is not None:
            mask = mask + self.slopes.to(device).float().view(1, -1, 1, 1) * kpos.float()
        return mask
