"""A dictionary (possibly nested, possibly with lists) whose leaves are datasets of equal length; items and
batches have the same nesting (reference: metaseq/data/nested_dictionary_dataset.py).

Leaves are addressed by dotted paths (``net_input.src_tokens``, list positions as ``[i]``); a batch is built by
asking each leaf dataset to collate its own column."""
from __future__ import annotations

from collections import OrderedDict

import torch
from torch.utils.data.dataloader import default_collate

from .base_dataset import BaseDataset


def _leaf_paths(tree):
    """Depth-first ``(dotted path, leaf)`` pairs; ``None`` leaves are dropped."""
    stack = [("", tree)]
    found = []
    while stack:
        path, node = stack.pop()
        if node is None:
            continue
        if isinstance(node, dict):
            children = [(f"{path}.{k}" if path else k, v) for k, v in node.items()]
        elif isinstance(node, list):
            children = [(f"{path}.[{i}]", v) for i, v in enumerate(node)]
        else:
            found.append((path, node))
            continue
        stack.extend(reversed(children))
    return found


def _rebuild(flat):
    root = OrderedDict()
    for path, value in flat.items():
        *parents, last = path.split(".")
        node = root
        for key in parents:
            if key[:1] == "[" and key[-1:] == "]":
                key = int(key[1:-1])
            node = node.setdefault(key, OrderedDict())
        node[last] = value
    return root


class NestedDictionaryDataset(BaseDataset):
    def __init__(self, defn, sizes=None):
        super().__init__()
        self.defn = OrderedDict(_leaf_paths(defn))
        self.sizes = list(sizes) if isinstance(sizes, (list, tuple)) else [sizes]
        lengths = set()
        for leaf in self.defn.values():
            if not isinstance(leaf, torch.utils.data.Dataset):
                raise ValueError("Expected Dataset but found: {}".format(leaf.__class__))
            if len(leaf) > 0:
                lengths.add(len(leaf))
        assert len(lengths) <= 1, "dataset lengths must match"
        self._len = lengths.pop() if lengths else 0

    def __len__(self):
        return self._len

    def __getitem__(self, index):
        return OrderedDict((path, leaf[index]) for path, leaf in self.defn.items())

    def collater(self, samples):
        if not samples:
            return {}
        batch = OrderedDict()
        for path, leaf in self.defn.items():
            column = [s[path] for s in samples]
            try:
                batch[path] = leaf.collater(column)
            except NotImplementedError:
                batch[path] = default_collate(column)
        return _rebuild(batch)

    def num_tokens(self, index):
        return max(s[index] for s in self.sizes)

    def size(self, index):
        per = tuple(s[index] for s in self.sizes)
        return per[0] if len(per) == 1 else per

    def _leaves_with(self, attr):
        return [leaf for leaf in self.defn.values() if getattr(leaf, attr, False)]

    @property
    def supports_prefetch(self):
        return bool(self._leaves_with("supports_prefetch"))

    def prefetch(self, indices):
        for leaf in self._leaves_with("supports_prefetch"):
            leaf.prefetch(indices)

    @property
    def can_reuse_epoch_itr_across_epochs(self):
        return all(leaf.can_reuse_epoch_itr_across_epochs for leaf in self.defn.values())

    def set_epoch(self, epoch):
        super().set_epoch(epoch)
        for leaf in self.defn.values():
            fn = getattr(leaf, "set_epoch", None)
            if fn is not None:
                fn(epoch)
