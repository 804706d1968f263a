"""Map-style language-modeling samples over a token-block dataset.

Each item pairs a block (``source``: the tokens shifted right by one) with its prediction target; a batch is
``{id, nsentences, ntokens, net_input: {src_tokens, src_lengths}, target}`` with right padding.  Behaviour
follows metaseq/data/monolingual_dataset.py:12-191: targets outside a smaller target vocabulary become ``unk``,
``add_bos_token`` prepends the beginning-of-sentence symbol or, for multilingual models, the language-id token
given as ``src_lang_idx`` / ``tgt_lang_idx``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from . import data_utils
from .base_dataset import BaseDataset

TokensOrList = Union[torch.Tensor, List[torch.Tensor]]


class _Padder:
    """Right-pads lists of 1-D token tensors into a ``[batch, length]`` matrix with one fixed set of options."""

    def __init__(self, pad_idx: int, eos_idx: int, fixed_pad_length: Optional[int], pad_to_bsz: Optional[int]):
        self.kw = dict(pad_idx=pad_idx, eos_idx=eos_idx, left_pad=False, pad_to_length=fixed_pad_length,
                       pad_to_bsz=pad_to_bsz)

    def __call__(self, rows: Sequence[torch.Tensor]) -> torch.Tensor:
        return data_utils.collate_tokens(list(rows), **self.kw)

    def field(self, samples, key: str):
        """One matrix for a tensor field; a list of matrices for a field that holds several tensors per sample."""
        first = samples[0][key]
        if isinstance(first, list):
            return [self([s[key][j] for s in samples]) for j in range(len(first))]
        return self([s[key] for s in samples])


def collate(samples, pad_idx, eos_idx, fixed_pad_length=None, pad_to_bsz=None):
    if not samples:
        return {}
    pad = _Padder(pad_idx, eos_idx, fixed_pad_length, pad_to_bsz)
    src_tokens = pad.field(samples, "source")
    lengths = [int(s["source"].numel()) for s in samples]
    batch = {
        "id": torch.tensor([s["id"] for s in samples], dtype=torch.long),
        "nsentences": len(samples),
        "ntokens": sum(lengths),
        "net_input": {"src_tokens": src_tokens, "src_lengths": torch.tensor(lengths, dtype=torch.long)},
    }
    # samples without a target of their own (plain blocks) are scored against their own tokens
    batch["target"] = src_tokens if samples[0]["target"] is None else pad.field(samples, "target")
    return batch


class MonolingualDataset(BaseDataset):
    def __init__(self, dataset, sizes, src_vocab, tgt_vocab=None, add_eos_for_other_targets=False, shuffle=False,
                 add_bos_token=False, fixed_pad_length=None, pad_to_bsz=None, src_lang_idx=None, tgt_lang_idx=None):
        super().__init__()
        self.dataset = dataset
        self.sizes = np.asarray(sizes)
        self.vocab = src_vocab
        self.tgt_vocab = src_vocab if tgt_vocab is None else tgt_vocab
        self.add_eos_for_other_targets = add_eos_for_other_targets
        self.shuffle = shuffle
        self.add_bos_token = add_bos_token
        self.fixed_pad_length = fixed_pad_length
        self.pad_to_bsz = pad_to_bsz
        # first token of source / target when ``add_bos_token``: a language id if given, else <s>
        self.src_lang_idx = src_lang_idx
        self.tgt_lang_idx = tgt_lang_idx
        self._clip_targets = len(self.tgt_vocab) != len(self.vocab)

    def __len__(self):
        return len(self.dataset)

    def __getitem__(self, index):
        item = self.dataset[index]
        if isinstance(item, tuple):  # TokenBlockDataset(include_targets=True): (source, future target, past target)
            source, target = item[0], self._filter_vocab(item[1])
        else:
            source, target = item, None
        source, target = self._maybe_add_bos(source, target)
        return {"id": index, "source": source, "target": target}

    def _filter_vocab(self, target: Optional[TokensOrList]) -> Optional[TokensOrList]:
        """Ids beyond the target vocabulary (it may be a truncated copy of the source one) map to ``unk``."""
        if target is None or not self._clip_targets:
            return target
        limit, unk = len(self.tgt_vocab), self.tgt_vocab.unk()

        def clip(t: torch.Tensor) -> torch.Tensor:
            return torch.where(t >= limit, torch.full_like(t, unk), t)

        return [clip(t) for t in target] if isinstance(target, list) else clip(target)

    def _maybe_add_bos(self, source, target):
        if not self.add_bos_token:
            return source, target
        first_src = self.src_lang_idx if self.src_lang_idx else self.vocab.bos()
        source = torch.cat([source.new_tensor([first_src]), source])
        if target is not None:
            first_tgt = self.tgt_lang_idx if self.tgt_lang_idx else self.tgt_vocab.bos()
            if isinstance(target, list):
                target = [torch.cat([t.new_tensor([first_tgt]), t]) for t in target]
            else:
                target = torch.cat([target.new_tensor([first_tgt]), target])
        return source, target

    def collater(self, samples):
        return collate(samples, self.vocab.pad(), self.vocab.eos(), self.fixed_pad_length, self.pad_to_bsz)

    # ----------------------------------------------------------------- sizes
    def num_tokens(self, index):
        return int(self.sizes[index])

    def num_tokens_vec(self, indices):
        return self.sizes[indices]

    def size(self, index):
        return int(self.sizes[index])

    def ordered_indices(self):
        """Shortest first; ties in random order when shuffling, in index order otherwise."""
        n = len(self)
        tie_break = np.random.permutation(n) if self.shuffle else np.arange(n)
        return np.lexsort((tie_break, self.sizes))

    # -------------------------------------------------------------- prefetch
    @property
    def supports_prefetch(self):
        return bool(getattr(self.dataset, "supports_prefetch", False))

    def prefetch(self, indices):
        self.dataset.prefetch(indices)
