"""Per-epoch random resampling of a dataset: ``ceil(len * size_ratio)`` indices drawn from
``RandomState([42, seed, epoch])``, with replacement iff the ratio exceeds 1 (or when asked),
optionally with per-item weights (reference: metaseq/data/resampling_dataset.py)."""
from __future__ import annotations

import logging

import numpy as np

from .base_dataset import BaseDataset

logger = logging.getLogger(__name__)


class ResamplingDataset(BaseDataset):
    def __init__(self, dataset, weights=None, replace=True, size_ratio=1.0, batch_by_size=True, seed=0, epoch=1):
        super().__init__()
        self.dataset = dataset
        if weights is not None:
            assert len(weights) == len(dataset)
            w = np.array(weights, dtype=np.float64)
            w /= w.sum()
            self.weights = w
        else:
            self.weights = None
        self.replace = replace
        assert size_ratio > 0.0
        if not self.replace:
            assert size_ratio <= 1.0
        self.actual_size = np.ceil(len(dataset) * size_ratio).astype(int)
        self.batch_by_size_flag = batch_by_size
        self.seed = seed
        self._cur_epoch = None
        self._cur_indices = None
        self.set_epoch(epoch)

    def __getitem__(self, index):
        return self.dataset[int(self._cur_indices[index])]

    def __len__(self):
        return int(self.actual_size)

    @property
    def sizes(self):
        if isinstance(self.dataset.sizes, list):
            return [s[self._cur_indices] for s in self.dataset.sizes]
        return self.dataset.sizes[self._cur_indices]

    def num_tokens(self, index):
        return self.dataset.num_tokens(self._cur_indices[index])

    def size(self, index):
        return self.dataset.size(self._cur_indices[index])

    def ordered_indices(self):
        if self.batch_by_size_flag:
            order = [np.arange(len(self)), self.sizes]
            return np.lexsort(order)
        return np.arange(len(self))

    def prefetch(self, indices):
        self.dataset.prefetch(self._cur_indices[indices])

    def collater(self, samples):
        return self.dataset.collater(samples)

    @property
    def can_reuse_epoch_itr_across_epochs(self):
        return False

    def set_epoch(self, epoch):
        logger.debug(f"ResamplingDataset.set_epoch: {epoch}")
        if hasattr(self.dataset, "set_epoch"):
            self.dataset.set_epoch(epoch)
        if epoch == self._cur_epoch:
            return
        self._cur_epoch = epoch
        rng = np.random.RandomState([42, self.seed % (2 ** 32), self._cur_epoch])
        self._cur_indices = rng.choice(len(self.dataset), int(self.actual_size), replace=self.replace,
                                       p=self.weights)
