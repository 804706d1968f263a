"""Round-robin partition of an iterable dataset across data-parallel ranks: out of every
group of ``num_shards`` consecutive items, rank ``shard_id`` keeps its own; a trailing
incomplete group is dropped (or completed with ``None`` when ``drop_last=False``).
Reference: metaseq/data/partitioned_streaming_dataset.py:43-54."""
from __future__ import annotations

import torch


class PartitionedStreamingDataset(torch.utils.data.IterableDataset):
    def __init__(self, dataset: torch.utils.data.IterableDataset, num_shards: int, shard_id: int,
                 drop_last: bool = True):
        super().__init__()
        self.dataset = dataset
        self.num_shards = num_shards
        self.shard_id = shard_id
        self.drop_last = drop_last
        assert isinstance(dataset, torch.utils.data.IterableDataset)
        assert num_shards > 0 and 0 <= shard_id < num_shards

    def set_epoch(self, epoch):
        if hasattr(self.dataset, "set_epoch"):
            self.dataset.set_epoch(epoch)

    def __iter__(self):
        group = []
        for x in self.dataset:
            group.append(x)
            if len(group) == self.num_shards:
                yield group[self.shard_id]
                group = []
        if group and not self.drop_last:
            yield group[self.shard_id] if self.shard_id < len(group) else None
