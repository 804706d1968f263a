"""Concatenation of map-style datasets with optional integer up-sampling ratios."""
from __future__ import annotations

import bisect

import numpy as np

from .base_dataset import BaseDataset


class ConcatDataset(BaseDataset):
    @staticmethod
    def cumsum(sequence, sample_ratios):
        r, s = [], 0
        for e, ratio in zip(sequence, sample_ratios):
            s += int(ratio * len(e))
            r.append(s)
        return r

    def __init__(self, datasets, sample_ratios=1):
        super().__init__()
        assert len(datasets) > 0, "datasets should not be an empty iterable"
        self.datasets = list(datasets)
        if isinstance(sample_ratios, int):
            sample_ratios = [sample_ratios] * len(self.datasets)
        self.sample_ratios = sample_ratios
        self.cumulative_sizes = self.cumsum(self.datasets, sample_ratios)
        self.real_sizes = [len(d) for d in self.datasets]

    def __len__(self):
        return self.cumulative_sizes[-1]

    def _locate(self, idx):
        ds = bisect.bisect_right(self.cumulative_sizes, idx)
        local = idx if ds == 0 else idx - self.cumulative_sizes[ds - 1]
        return ds, local % self.real_sizes[ds]

    def __getitem__(self, idx):
        ds, local = self._locate(idx)
        return self.datasets[ds][local]

    def collater(self, samples, **extra):
        if hasattr(self.datasets[0], "collater"):
            return self.datasets[0].collater(samples, **extra)
        from torch.utils.data.dataloader import default_collate

        return default_collate(samples, **extra)

    def size(self, idx):
        ds, local = self._locate(idx)
        return self.datasets[ds].size(local)

    def num_tokens(self, idx):
        return np.max(self.size(idx))

    @property
    def sizes(self):
        out = []
        for ds, sr in zip(self.datasets, self.sample_ratios):
            out.append(np.tile(ds.sizes, sr) if isinstance(ds.sizes, np.ndarray) else np.tile(ds.sizes[0], sr))
        return np.concatenate(out)

    @property
    def supports_prefetch(self):
        return all(getattr(d, "supports_prefetch", False) for d in self.datasets)

    def ordered_indices(self):
        return np.argsort(self.sizes)

    def attr(self, attr: str, index: int):
        """The attribute as the member dataset that holds ``index`` has it."""
        ds, _ = self._locate(index)
        return getattr(self.datasets[ds], attr, None)

    def prefetch(self, indices):
        """Hands every member the indices that fall into it, in its own numbering."""
        start = 0
        for end, real, ds in zip(self.cumulative_sizes, self.real_sizes, self.datasets):
            if getattr(ds, "supports_prefetch", False):
                ds.prefetch([(i - start) % real for i in indices if start <= i < end])
            start = end

    def ordered_indices_per_dataset(self):
        """Every member's ordered index vectors, shifted into this dataset's numbering."""
        out, start = [], 0
        for end, ds in zip(self.cumulative_sizes, self.datasets):
            for idx in ds.ordered_indices_per_dataset():
                out.append(np.asarray(idx) + start)
            start = end
        return out

    def set_epoch(self, epoch):
        for d in self.datasets:
            if hasattr(d, "set_epoch"):
                d.set_epoch(epoch)
