"""Dataset that forwards everything to a wrapped dataset (reference: metaseq/data/base_wrapper_dataset.py).

Subclasses override only what they change; every other dataset-protocol method is generated below as a
plain delegation to ``self.dataset``."""
from __future__ import annotations

from torch.utils.data.dataloader import default_collate

from .base_dataset import BaseDataset

_DELEGATED_METHODS = ("num_tokens", "num_tokens_vec", "size", "ordered_indices", "attr", "prefetch",
                      "filter_indices_by_size", "batch_by_size")
_DELEGATED_PROPERTIES = ("sizes", "can_reuse_epoch_itr_across_epochs")


class BaseWrapperDataset(BaseDataset):
    def __init__(self, dataset):
        super().__init__()
        self.dataset = dataset

    def __len__(self):
        return len(self.dataset)

    def __getitem__(self, index):
        return self.dataset[index]

    def collater(self, samples):
        inner = getattr(self.dataset, "collater", None)
        return inner(samples) if inner is not None else default_collate(samples)

    @property
    def supports_prefetch(self):
        return bool(getattr(self.dataset, "supports_prefetch", False))

    def get_batch_shapes(self):
        inner = getattr(self.dataset, "get_batch_shapes", None)  # the wrapped object may be a plain sequence
        return inner() if inner is not None else None

    def set_epoch(self, epoch):
        super().set_epoch(epoch)
        inner = getattr(self.dataset, "set_epoch", None)
        if inner is not None:
            inner(epoch)


def _method(name):
    def call(self, *args, **kwargs):
        return getattr(self.dataset, name)(*args, **kwargs)

    call.__name__ = name
    return call


for _n in _DELEGATED_METHODS:
    setattr(BaseWrapperDataset, _n, _method(_n))
for _n in _DELEGATED_PROPERTIES:
    setattr(BaseWrapperDataset, _n, property(lambda self, _n=_n: getattr(self.dataset, _n)))
