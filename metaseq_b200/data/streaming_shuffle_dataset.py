"""Shuffles a map-style dataset per epoch and exposes it as an iterable, splitting the
order across DataLoader workers."""
from __future__ import annotations

import numpy as np
import torch

from metaseq_b200.utils import numpy_seed


class StreamingShuffleDataset(torch.utils.data.IterableDataset):
    def __init__(self, dataset: torch.utils.data.Dataset, seed: int):
        super().__init__()
        self.dataset = dataset
        self.seed = seed
        assert len(dataset) > 0
        self.indices = None

    def set_epoch(self, epoch):
        with numpy_seed(self.seed, epoch):
            self.indices = np.random.permutation(len(self.dataset))
        if hasattr(self.dataset, "set_epoch"):
            self.dataset.set_epoch(epoch)

    def __iter__(self):
        assert self.indices is not None, "must call StreamingShuffleDataset.set_epoch before iteration"
        info = torch.utils.data.get_worker_info()
        indices = self.indices
        if info is not None and info.num_workers > 1:
            indices = np.array_split(indices, info.num_workers)[info.id]
        for i in indices:
            yield self.dataset[int(i)]
