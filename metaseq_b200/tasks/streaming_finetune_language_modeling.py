"""Fine-tuning on (source, target) JSONL pairs: both sides are tokenised, concatenated into
one sequence and the loss is taken on the target part only (the source positions of the
target tensor are pad) (reference: metaseq/tasks/streaming_finetune_language_modeling.py:31-149)."""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Any, Dict, List

import torch

from metaseq_b200.data import ConcatDataset, DocumentToSequenceDataset, JsonlDataset, data_utils
from metaseq_b200.tasks import register_task
from metaseq_b200.tasks.streaming_language_modeling import StreamingLanguageModelingConfig, StreamingLanguageModelingTask

logger = logging.getLogger(__name__)


@dataclass
class StreamingFinetuneLanguageModelingConfig(StreamingLanguageModelingConfig):
    pass


@register_task("streaming_finetune_language_modeling", dataclass=StreamingFinetuneLanguageModelingConfig)
class StreamingFinetuneLanguageModelingTask(StreamingLanguageModelingTask):
    def _tokenize_src_tgt_json(self, json):
        src = json["src"].rstrip(" ")
        tgt = json["tgt"].rstrip()
        full = torch.LongTensor(self.tokenizer.encode(" ".join([src, tgt])).ids + [self.eod])
        src_len = len(self.tokenizer.encode(src).ids)
        tgt_tokens = torch.clone(full)
        tgt_tokens[:src_len] = self.dictionary.pad_index
        return full, tgt_tokens

    def load_dataset(self, split: str, epoch=1, combine=False, **kwargs):
        base = os.path.join(self.args.data, split)
        files = sorted(f for f in os.listdir(base) if f.endswith(".jsonl"))
        if not files:  # sharded layout
            shard = self.get_shard_str(epoch, split)
            base = os.path.join(base, shard)
            files = sorted(f for f in os.listdir(base) if f.endswith(".jsonl"))
        datasets = [JsonlDataset(os.path.join(base, f), tokenizer=self._tokenize_src_tgt_json, epoch=epoch)
                    for f in files]
        dataset = ConcatDataset(datasets) if len(datasets) > 1 else datasets[0]
        self.datasets[split] = DocumentToSequenceDataset(
            dataset, block_size=self.args.tokens_per_sample + 1,
            break_mode=self.args.sample_break_mode if self.args.sample_break_mode not in (None, "none") else "complete",
            drop_last=(split == "train"), padding_idx=self.source_dictionary.pad(), seed=self.args.seed,
            source_target=True)
        return self.datasets[split]

    def _collate_fn(self, items: List[Dict[str, Any]]):
        if len(items) > 0 and items[0] is None:
            return {}
        items = [x for x in items if x is not None]
        pad = self.source_dictionary.pad()
        src = data_utils.collate_tokens([x["src_block"] for x in items], pad_idx=pad, pad_to_bsz=self.args.batch_size)
        tgt = data_utils.collate_tokens([x["tgt_block"] for x in items], pad_idx=pad, pad_to_bsz=self.args.batch_size)
        input = src[:, :-1].contiguous()
        target = tgt[:, 1:].contiguous()
        ids = torch.cat([x["ids"] for x in items])
        return {
            "id": ids,
            "net_input": {"src_tokens": input},
            "target": target,
            "nsentences": input.size(0),
            "ntokens": int(input.ne(pad).sum()),
            "ntokens_target": int(target.ne(pad).sum()),
        }
