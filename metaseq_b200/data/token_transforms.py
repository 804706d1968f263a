"""Per-item token edits: append / prepend / strip a token, and length bookkeeping datasets
(reference: metaseq/data/{append_token,prepend_token,strip_token,numel,id,list,pad,sort,shorten}_dataset.py)."""
from __future__ import annotations

import numpy as np
import torch

from . import data_utils
from .base_dataset import BaseDataset
from .base_wrapper_dataset import BaseWrapperDataset


class AppendTokenDataset(BaseWrapperDataset):
    def __init__(self, dataset, token=None):
        super().__init__(dataset)
        self.token = token
        self._sizes = np.array(dataset.sizes) + 1 if token is not None else dataset.sizes

    def __getitem__(self, idx):
        item = self.dataset[idx]
        if self.token is not None:
            item = torch.cat([item, item.new([self.token])])
        return item

    @property
    def sizes(self):
        return self._sizes

    def num_tokens(self, index):
        return self.dataset.num_tokens(index) + (1 if self.token is not None else 0)

    def size(self, index):
        return self.dataset.size(index) + (1 if self.token is not None else 0)


class PrependTokenDataset(BaseWrapperDataset):
    def __init__(self, dataset, token=None):
        super().__init__(dataset)
        self.token = token
        self._sizes = np.array(dataset.sizes) + 1 if token is not None else dataset.sizes

    def __getitem__(self, idx):
        item = self.dataset[idx]
        if self.token is not None:
            item = torch.cat([item.new([self.token]), item])
        return item

    @property
    def sizes(self):
        return self._sizes

    def num_tokens(self, index):
        return self.dataset.num_tokens(index) + (1 if self.token is not None else 0)

    def size(self, index):
        return self.dataset.size(index) + (1 if self.token is not None else 0)


class StripTokenDataset(BaseWrapperDataset):
    """Removes leading and trailing occurrences of ``id_to_strip``."""

    def __init__(self, dataset, id_to_strip):
        super().__init__(dataset)
        self.id_to_strip = id_to_strip

    def __getitem__(self, index):
        item = self.dataset[index]
        while len(item) > 0 and item[-1] == self.id_to_strip:
            item = item[:-1]
        while len(item) > 0 and item[0] == self.id_to_strip:
            item = item[1:]
        return item


class NumelDataset(BaseWrapperDataset):
    def __init__(self, dataset, reduce=False):
        super().__init__(dataset)
        self.reduce = reduce

    def __getitem__(self, index):
        item = self.dataset[index]
        return torch.numel(item) if torch.is_tensor(item) else np.size(item)

    def collater(self, samples):
        return sum(samples) if self.reduce else torch.tensor(samples)


class IdDataset(BaseDataset):
    def __getitem__(self, index):
        return index

    def __len__(self):
        return 0

    def collater(self, samples):
        return torch.tensor(samples)


class ListDataset(BaseWrapperDataset):
    def __init__(self, dataset, sizes=None):
        super().__init__(dataset)
        self._sizes = sizes

    def __iter__(self):
        for x in self.dataset:
            yield x

    def collater(self, samples):
        return samples

    @property
    def sizes(self):
        return self._sizes

    def num_tokens(self, index):
        return self.sizes[index]

    def size(self, index):
        return self.sizes[index]

    def set_epoch(self, epoch):
        pass


class PadDataset(BaseWrapperDataset):
    def __init__(self, dataset, pad_idx, left_pad):
        super().__init__(dataset)
        self.pad_idx = pad_idx
        self.left_pad = left_pad

    def collater(self, samples):
        return data_utils.collate_tokens(samples, self.pad_idx, left_pad=self.left_pad)


class LeftPadDataset(PadDataset):
    def __init__(self, dataset, pad_idx):
        super().__init__(dataset, pad_idx, left_pad=True)


class RightPadDataset(PadDataset):
    def __init__(self, dataset, pad_idx):
        super().__init__(dataset, pad_idx, left_pad=False)


class MultiplePadDataset(BaseWrapperDataset):
    """Items and batches right-padded to the next multiple of ``multiple`` (metaseq/data/pad_dataset.py:37-76)."""

    def __init__(self, dataset, pad_idx, multiple):
        super().__init__(dataset)
        self.pad_idx = pad_idx
        self.multiple = int(multiple)

    def _round_up(self, n: int) -> int:
        return -(-n // self.multiple) * self.multiple

    def __getitem__(self, index):
        item = self.dataset[index]
        extra = self._round_up(item.numel()) - item.numel()
        return item if extra == 0 else torch.cat([item, item.new_full((extra,), self.pad_idx)])

    def collater(self, samples):
        longest = max(s.size(0) for s in samples)
        return data_utils.collate_tokens(samples, self.pad_idx, left_pad=False, pad_to_length=self._round_up(longest))


class SortDataset(BaseWrapperDataset):
    """Orders indices by one or more keys (last key is the primary one, as in ``np.lexsort``)."""

    def __init__(self, dataset, sort_order):
        super().__init__(dataset)
        if not isinstance(sort_order, (list, tuple)):
            sort_order = [sort_order]
        self.sort_order = sort_order
        assert all(len(so) == len(dataset) for so in sort_order)

    def ordered_indices(self):
        return np.lexsort(self.sort_order)


class TruncateDataset(BaseWrapperDataset):
    """Keeps the first ``truncation_length`` tokens of every item."""

    def __init__(self, dataset, truncation_length):
        super().__init__(dataset)
        assert truncation_length is not None
        self.truncation_length = truncation_length

    def __getitem__(self, index):
        item = self.dataset[index]
        if item.size(0) > self.truncation_length:
            item = item[: self.truncation_length]
        return item

    @property
    def sizes(self):
        return np.minimum(self.dataset.sizes, self.truncation_length)


class RandomCropDataset(TruncateDataset):
    """Keeps a window of ``truncation_length`` tokens whose start depends on (seed, epoch, index)."""

    def __init__(self, dataset, truncation_length, seed=1):
        super().__init__(dataset, truncation_length)
        self.seed = seed
        self.epoch = 0

    @property
    def can_reuse_epoch_itr_across_epochs(self):
        return True

    def set_epoch(self, epoch, **unused):
        super().set_epoch(epoch)
        self.epoch = epoch

    def __getitem__(self, index):
        with data_utils.numpy_seed(self.seed, self.epoch, index):
            item = self.dataset[index]
            excess = item.size(0) - self.truncation_length
            if excess > 0:
                start = np.random.randint(0, excess)
                item = item[start:start + self.truncation_length]
            return item


def maybe_shorten_dataset(dataset, split, shorten_data_split_list, shorten_method, tokens_per_sample, seed):
    truncate_split = split in shorten_data_split_list.split(",") or len(shorten_data_split_list) == 0
    if shorten_method == "truncate" and truncate_split:
        dataset = TruncateDataset(dataset, tokens_per_sample)
    elif shorten_method == "random_crop" and truncate_split:
        dataset = RandomCropDataset(dataset, tokens_per_sample, seed)
    return dataset
