"""A map-style dataset served as a stream in a new random order every epoch (reference:
metaseq/data/streaming_shuffle_dataset.py).  The order is a function of ``(seed, epoch)`` alone, so every rank and
every restart sees the same one; data-loader workers take contiguous pieces of it."""
from __future__ import annotations

import numpy as np
import torch

from metaseq_b200.utils import numpy_seed


class StreamingShuffleDataset(torch.utils.data.IterableDataset):
    def __init__(self, dataset: torch.utils.data.Dataset, seed: int):
        super().__init__()
        assert len(dataset) > 0
        self.dataset, self.seed = dataset, seed
        self.indices = None  # drawn by set_epoch

    def set_epoch(self, epoch):
        inner = getattr(self.dataset, "set_epoch", None)
        with numpy_seed(self.seed, epoch):
            self.indices = np.random.permutation(len(self.dataset))
        if inner is not None:
            inner(epoch)

    def _my_share(self) -> np.ndarray:
        worker = torch.utils.data.get_worker_info()
        if worker is None or worker.num_workers <= 1:
            return self.indices
        return np.array_split(self.indices, worker.num_workers)[worker.id]

    def __iter__(self):
        assert self.indices is not None, "must call StreamingShuffleDataset.set_epoch before iteration"
        return (self.dataset[int(i)] for i in self._my_share())
