"""Per-epoch random resampling of a dataset: ``ceil(len * size_ratio)`` indices drawn from
``RandomState([42, seed, epoch])``, with replacement iff the ratio exceeds 1 (or when asked),
optionally with per-item weights (reference: metaseq/data/resampling_dataset.py)."""
from __future__ import annotations

import logging

import numpy as np

from .base_dataset import BaseDataset

logger = logging.getLogger(__name__)


class ResamplingDataset(BaseDataset):
    """``dataset[i]`` of this wrapper is ``dataset[draw[i]]`` where ``draw`` is redrawn for every epoch.

    ``weights``: one non-negative number per item of ``dataset`` (normalised here); ``None`` draws uniformly.
    ``size_ratio``: length of the wrapper relative to ``dataset`` (must be <= 1 without replacement).
    ``batch_by_size``: whether ``ordered_indices`` sorts by sample size (stable) or keeps the drawn order."""

    def __init__(self, dataset, weights=None, replace=True, size_ratio=1.0, batch_by_size=True, seed=0, epoch=1):
        super().__init__()
        assert size_ratio > 0.0 and (replace or size_ratio <= 1.0)
        self.dataset, self.replace, self.seed = dataset, replace, seed
        self.weights = None
        if weights is not None:
            assert len(weights) == len(dataset)
            self.weights = np.asarray(weights, dtype=np.float64) / float(np.sum(weights))
        self.actual_size = int(np.ceil(len(dataset) * size_ratio))
        self.batch_by_size_flag = batch_by_size
        self._cur_epoch, self._cur_indices = None, None
        self.set_epoch(epoch)

    # -- the draw ----------------------------------------------------------------------------------
    def set_epoch(self, epoch):
        inner = getattr(self.dataset, "set_epoch", None)
        if inner is not None:
            inner(epoch)
        if epoch != self._cur_epoch:
            logger.debug(f"ResamplingDataset.set_epoch: {epoch}")
            self._cur_epoch = epoch
            rng = np.random.RandomState([42, self.seed % (2 ** 32), epoch])  # same draw for the same (seed, epoch)
            self._cur_indices = rng.choice(len(self.dataset), self.actual_size, replace=self.replace, p=self.weights)

    @property
    def can_reuse_epoch_itr_across_epochs(self):
        return False  # every epoch has other items

    # -- everything else goes through the draw -----------------------------------------------------
    def __len__(self):
        return self.actual_size

    def __getitem__(self, index):
        return self.dataset[int(self._cur_indices[index])]

    def size(self, index):
        return self.dataset.size(self._cur_indices[index])

    def num_tokens(self, index):
        return self.dataset.num_tokens(self._cur_indices[index])

    @property
    def sizes(self):
        inner = self.dataset.sizes
        return [s[self._cur_indices] for s in inner] if isinstance(inner, list) else inner[self._cur_indices]

    def ordered_indices(self):
        positions = np.arange(len(self))
        return np.lexsort([positions, self.sizes]) if self.batch_by_size_flag else positions

    def prefetch(self, indices):
        self.dataset.prefetch(self._cur_indices[indices])

    def collater(self, samples):
        return self.dataset.collater(samples)
