"""Language-modeling samples ``{id, net_input: {src_tokens, src_lengths}, target, ntokens}`` over a token
block dataset (reference: metaseq/data/monolingual_dataset.py:12-191)."""
from __future__ import annotations

import numpy as np
import torch

from . import data_utils
from .base_dataset import BaseDataset


def collate(samples, pad_idx, eos_idx, fixed_pad_length=None, pad_to_bsz=None):
    if len(samples) == 0:
        return {}

    def merge(key, is_list=False):
        if is_list:
            return [data_utils.collate_tokens([s[key][i] for s in samples], pad_idx, eos_idx, left_pad=False,
                                              pad_to_length=fixed_pad_length, pad_to_bsz=pad_to_bsz)
                    for i in range(len(samples[0][key]))]
        return data_utils.collate_tokens([s[key] for s in samples], pad_idx, eos_idx, left_pad=False,
                                         pad_to_length=fixed_pad_length, pad_to_bsz=pad_to_bsz)

    src_tokens = merge("source")
    if samples[0]["target"] is not None:
        target = merge("target", is_list=isinstance(samples[0]["target"], list))
    else:
        target = src_tokens
    return {
        "id": torch.LongTensor([s["id"] for s in samples]),
        "nsentences": len(samples),
        "ntokens": sum(len(s["source"]) for s in samples),
        "net_input": {"src_tokens": src_tokens, "src_lengths": torch.LongTensor([s["source"].numel() for s in samples])},
        "target": target,
    }


class MonolingualDataset(BaseDataset):
    def __init__(self, dataset, sizes, src_vocab, tgt_vocab=None, add_eos_for_other_targets=False, shuffle=False,
                 add_bos_token=False, fixed_pad_length=None, pad_to_bsz=None, src_lang_idx=None, tgt_lang_idx=None):
        super().__init__()
        self.dataset = dataset
        self.sizes = np.array(sizes)
        self.vocab = src_vocab
        self.tgt_vocab = tgt_vocab or src_vocab
        self.add_eos_for_other_targets = add_eos_for_other_targets
        self.shuffle = shuffle
        self.add_bos_token = add_bos_token
        self.fixed_pad_length = fixed_pad_length
        self.pad_to_bsz = pad_to_bsz
        self.src_lang_idx = src_lang_idx
        self.tgt_lang_idx = tgt_lang_idx

    def __getitem__(self, index):
        # the wrapped TokenBlockDataset(include_targets=True) yields (source, future target, past target);
        # a plain item is used both as source and (shifted by the criterion's caller) as target
        item = self.dataset[index]
        if isinstance(item, tuple):
            source, target, _ = item
        else:
            source, target = item, None
        source, target = self._maybe_add_bos(source, target)
        return {"id": index, "source": source, "target": target}

    def __len__(self):
        return len(self.dataset)

    def _maybe_add_bos(self, source, target):
        if self.add_bos_token:
            source = torch.cat([source.new([self.vocab.bos()]), source])
            if target is not None:
                target = torch.cat([target.new([self.tgt_vocab.bos()]), target])
        return source, target

    def num_tokens_vec(self, indices):
        return self.sizes[indices]

    def collater(self, samples):
        return collate(samples, self.vocab.pad(), self.vocab.eos(), self.fixed_pad_length, self.pad_to_bsz)

    def num_tokens(self, index):
        return int(self.sizes[index])

    def size(self, index):
        return int(self.sizes[index])

    def ordered_indices(self):
        if self.shuffle:
            order = [np.random.permutation(len(self))]
        else:
            order = [np.arange(len(self))]
        order.append(self.sizes)
        return np.lexsort(order)

    @property
    def supports_prefetch(self):
        return getattr(self.dataset, "supports_prefetch", False)

    def prefetch(self, indices):
        self.dataset.prefetch(indices)
