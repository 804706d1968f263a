"""Synthetic token documents for benchmarks and tests: token ids uniform in
``[4, vocab_size)`` and document lengths geometric with a given mean, both from a seed; each
document ends with EOS.  Deterministic per index, so it behaves like a tokenised corpus of
``num_docs`` documents without touching the filesystem."""
from __future__ import annotations

import numpy as np
import torch


class SyntheticDocumentDataset(torch.utils.data.Dataset):
    def __init__(self, num_docs: int, vocab_size: int, mean_len: float, seed: int = 1, eos: int = 2,
                 first_token: int = 4, max_len: int = 1 << 20):
        self.num_docs = num_docs
        self.vocab_size = vocab_size
        self.seed = seed
        self.eos = eos
        self.first_token = first_token
        rng = np.random.default_rng([seed, 7919])
        self.lengths = np.minimum(rng.geometric(1.0 / max(mean_len, 1.0), size=num_docs), max_len).astype(np.int64)

    def __len__(self):
        return self.num_docs

    def __getitem__(self, idx):
        n = int(self.lengths[idx])
        rng = np.random.default_rng([self.seed, int(idx)])
        toks = rng.integers(self.first_token, self.vocab_size, size=n, dtype=np.int64)
        toks[-1] = self.eos
        return torch.from_numpy(toks)
