"""Adaptive softmax (Grave et al., "Efficient softmax approximation for GPUs"): the vocabulary is cut into a
frequent head and rarer tail clusters; the head predicts the frequent words plus one logit per cluster, and each
tail uses a projection to a smaller dimension (reference: metaseq/modules/adaptive_softmax.py).  The OPT recipes do
not use it; it is provided for models configured with ``--adaptive-softmax-cutoff``."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from .quant_noise import quant_noise


class TiedLinear(nn.Module):
    def __init__(self, weight, transpose):
        super().__init__()
        self.weight, self.transpose = weight, transpose

    def forward(self, input):
        return F.linear(input, self.weight.t() if self.transpose else self.weight)


class TiedHeadModule(nn.Module):
    """Head of an adaptive softmax whose frequent-word logits reuse the first band of an adaptive input embedding:
    ``[word logits | cluster logits]``, the cluster logits from a projection of their own.  ``weights`` is the
    band's (embedding weight, projection weight) pair (metaseq/modules/adaptive_softmax.py:26-55)."""

    def __init__(self, weights, input_dim: int, num_classes: int, q_noise: float = 0, qn_block_size: int = 8):
        super().__init__()
        tied_emb, _ = weights
        self.num_words, emb_dim = tied_emb.size()
        words = quant_noise(TiedLinear(tied_emb, transpose=False), q_noise, qn_block_size)
        if input_dim != emb_dim:
            words = nn.Sequential(quant_noise(nn.Linear(input_dim, emb_dim, bias=False), q_noise, qn_block_size), words)
        self.word_proj = words
        self.class_proj = quant_noise(nn.Linear(input_dim, num_classes, bias=False), q_noise, qn_block_size)
        self.out_dim = self.num_words + num_classes

    def forward(self, input):
        flat = input.reshape(-1, input.size(-1))
        return torch.cat([self.word_proj(flat), self.class_proj(flat)], dim=1)


class AdaptiveSoftmax(nn.Module):
    def __init__(self, vocab_size: int, input_dim: int, cutoff: List[int], dropout: float, factor: float = 4.0,
                 adaptive_inputs=None, tie_proj: bool = False, q_noise: float = 0, qn_block_size: int = 8):
        super().__init__()
        cutoff = list(cutoff)
        if vocab_size > cutoff[-1]:
            cutoff = cutoff + [vocab_size]
        else:
            assert vocab_size == cutoff[-1], "cannot specify cutoff larger than vocab size"
        self.vocab_size, self.cutoff, self.input_dim, self.factor = vocab_size, cutoff, input_dim, factor
        self.dropout = nn.Dropout(dropout)
        n_clusters = len(cutoff) - 1
        if adaptive_inputs is None:
            self.head = quant_noise(nn.Linear(input_dim, cutoff[0] + n_clusters, bias=False), q_noise, qn_block_size)
        else:
            self.head = TiedHeadModule(adaptive_inputs.weights_for_band(0), input_dim, n_clusters, q_noise, qn_block_size)
        self.tail = nn.ModuleList()
        for i in range(n_clusters):
            dim = int(input_dim // factor ** (i + 1))
            size = cutoff[i + 1] - cutoff[i]
            tied_emb, tied_proj = adaptive_inputs.weights_for_band(i + 1) if adaptive_inputs is not None else (None, None)
            if tied_proj is not None and tie_proj:
                proj = quant_noise(TiedLinear(tied_proj, transpose=True), q_noise, qn_block_size)
            elif tied_proj is not None:
                proj = quant_noise(nn.Linear(tied_proj.size(0), tied_proj.size(1), bias=False), q_noise, qn_block_size)
            else:
                proj = quant_noise(nn.Linear(input_dim, dim, bias=False), q_noise, qn_block_size)
            if tied_emb is None:
                out = quant_noise(nn.Linear(dim, size, bias=False), q_noise, qn_block_size)
            else:
                out = quant_noise(TiedLinear(tied_emb, transpose=False), q_noise, qn_block_size)
            self.tail.append(nn.Sequential(proj, nn.Dropout(dropout), out))
        self.lsm = nn.LogSoftmax(dim=1)
        self.apply(self._init)
        # state dicts carry the layout version (the reference's checkpoints have this key; older layouts are refused)
        self.register_buffer("version", torch.LongTensor([1]))

    def upgrade_state_dict_named(self, state_dict, name):
        if name + ".version" not in state_dict:
            raise Exception("This version of the model is no longer supported")

    @staticmethod
    def _init(m):
        if isinstance(m, nn.Linear):
            nn.init.xavier_uniform_(m.weight)

    def adapt_target(self, target):
        """Head targets (tail words replaced by their cluster's logit index) and per-cluster (row indices, targets)."""
        target = target.view(-1)
        head_target = target.clone()
        tails, rows = [], []
        for i in range(len(self.cutoff) - 1):
            in_cluster = target.ge(self.cutoff[i]) & target.lt(self.cutoff[i + 1])
            head_target[in_cluster] = self.cutoff[0] + i
            if in_cluster.any():
                rows.append(in_cluster.nonzero(as_tuple=False).squeeze(1))
                tails.append(target[in_cluster] - self.cutoff[i])
            else:
                rows.append(None)
                tails.append(None)
        return [head_target] + tails, rows

    def forward(self, input, target):
        """Returns (list of logits, list of targets): entry 0 is the head, entry i+1 cluster i (or None)."""
        input = self.dropout(input.contiguous().view(-1, input.size(-1)))
        new_target, rows = self.adapt_target(target)
        output = [self.head(input)]
        for i, idx in enumerate(rows):
            output.append(None if idx is None else self.tail[i](input.index_select(0, idx)))
        return output, new_target

    def get_log_prob(self, input, target: Optional[torch.Tensor]):
        """Full-vocabulary log-probabilities ``[B, T, V]`` (used at inference)."""
        bsz, length, dim = input.size()
        input = input.contiguous().view(-1, dim)
        head_lp = self.lsm(self.head(input))
        out = input.new_zeros(input.size(0), self.vocab_size)
        head_size = self.cutoff[0]
        out[:, :head_size] = head_lp[:, :head_size]
        for i in range(len(self.tail)):
            lo, hi = self.cutoff[i], self.cutoff[i + 1]
            out[:, lo:hi] = self.lsm(self.tail[i](input)) + head_lp[:, head_size + i, None]
        return out.view(bsz, length, -1)
