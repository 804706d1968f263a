"""``dummy_lm``: a fixed synthetic batch repeated forever, for benchmarking the training step
without a data pipeline (reference: metaseq/benchmark/dummy_lm.py:35-126; selected by
``--benchmark`` in the launcher)."""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from metaseq_b200.data import BaseDataset, Dictionary
from metaseq_b200.dataclass.configs import MetaseqDataclass, opt
from metaseq_b200.tasks import BaseTask, register_task

logger = logging.getLogger(__name__)


@dataclass
class DummyLMConfig(MetaseqDataclass):
    dict_size: int = opt(50272, "vocabulary size (padded to a multiple of 8)")
    dataset_size: int = opt(100000, "number of synthetic samples per epoch")
    tokens_per_sample: int = opt(512, "max number of total tokens over all segments per sample")
    add_bos_token: bool = opt(False, "prepend beginning of sentence token (<s>)")
    batch_size: Optional[int] = opt(None, link="dataset.batch_size")
    max_tokens: Optional[int] = opt(None, link="dataset.max_tokens")
    max_target_positions: Optional[int] = opt(None, "max number of tokens in the target sequence")
    random_tokens: bool = opt(True, "uniform random token ids (seeded) instead of an arange ramp")
    seed: int = opt(1, link="common.seed")


@register_task("dummy_lm", dataclass=DummyLMConfig)
class DummyLMTask(BaseTask):
    def __init__(self, cfg):
        super().__init__(cfg)
        self.dictionary = Dictionary.synthetic(cfg.dict_size)
        self.dictionary.pad_to_multiple_(8)
        logger.info(f"dictionary: {len(self.dictionary)} types")
        T = cfg.tokens_per_sample
        if getattr(cfg, "random_tokens", True):
            g = torch.Generator().manual_seed(int(getattr(cfg, "seed", 1)))
            seq = torch.randint(self.dictionary.nspecial, len(self.dictionary), (T + 1,), generator=g)
        else:
            seq = torch.arange(T + 1) + self.dictionary.pad() + 1
        self.dummy_src = seq[:-1]
        self.dummy_tgt = seq[1:]

    def load_dataset(self, split, epoch=1, combine=False, **kwargs):
        if self.cfg.batch_size is not None:
            bsz = self.cfg.batch_size
        else:
            bsz = max(1, self.cfg.max_tokens // self.cfg.tokens_per_sample)
        g = torch.Generator().manual_seed(int(getattr(self.cfg, "seed", 1)) + 1)
        if getattr(self.cfg, "random_tokens", True):
            blocks = torch.randint(self.dictionary.nspecial, len(self.dictionary),
                                   (bsz, self.cfg.tokens_per_sample + 1), generator=g)
            src, tgt = blocks[:, :-1].contiguous(), blocks[:, 1:].contiguous()
        else:
            src = torch.stack([self.dummy_src for _ in range(bsz)])
            tgt = torch.stack([self.dummy_tgt for _ in range(bsz)])
        self.datasets[split] = DummyDataset(
            {
                "id": 1,
                "net_input": {"src_tokens": src},
                "target": tgt,
                "nsentences": bsz,
                "ntokens": bsz * self.cfg.tokens_per_sample,
            },
            num_items=self.cfg.dataset_size,
            item_size=self.cfg.tokens_per_sample,
        )

    @property
    def source_dictionary(self):
        return self.dictionary

    @property
    def target_dictionary(self):
        return self.dictionary

    def max_positions(self):
        return self.cfg.tokens_per_sample


class DummyDataset(BaseDataset):
    """``num_items`` items of ``item_size`` tokens each; whatever indices a batch is made of, collating them yields
    the one prepared ``batch``."""

    supports_prefetch = False

    def __init__(self, batch, num_items: int, item_size: int):
        super().__init__()
        self.batch, self.num_items, self.item_size = batch, int(num_items), int(item_size)
        self.sizes = np.full(self.num_items, self.item_size, dtype=np.int64)

    def __len__(self):
        return self.num_items

    def __getitem__(self, index):
        return index

    def collater(self, samples):
        return self.batch

    def num_tokens(self, index):
        return self.item_size

    size = num_tokens

    def ordered_indices(self):
        return np.arange(self.num_items)
