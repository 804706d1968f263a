"""Streaming language-modeling task: JSONL corpora (or synthetic documents) -> BPE ->
EOS-terminated documents -> packed blocks of ``tokens_per_sample + 1`` -> batches sharded
over the data-parallel group.

Behaviour follows the reference (metaseq/tasks/streaming_language_modeling.py:153-577):
the dictionary is built from the tokenizer with specials ``<s> <pad> </s> <unk>`` at 0..3
(:195-210); every document is ``ids(text.rstrip()) + </s>`` (:264-270); one epoch reads one
shard directory ``<data>/<split>/<NN>/*.jsonl`` (:350-364); corpora are resampled with
temperature ``alpha`` (:272-348); the collater emits ``{id, net_input.src_tokens, target,
nsentences, ntokens}`` with input ``block[:-1]`` and target ``block[1:]`` (:448-478); the
iterator shuffles through a buffer of ``10 * batch_size * num_shards`` sequences and
partitions round-robin over data-parallel ranks (:483-569).

``--synthetic-data N`` replaces the corpus by N seeded synthetic documents (uniform token
ids, geometric lengths) so that benchmarks and tests need no files or tokenizer.
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from metaseq_b200 import utils
from metaseq_b200.data import (
    ConcatDataset,
    Dictionary,
    DocumentToSequenceDataset,
    JsonlDataset,
    PartitionedStreamingDataset,
    ResamplingDataset,
    SyntheticDocumentDataset,
    data_utils,
    iterators,
)
from metaseq_b200.dataclass.configs import MetaseqDataclass, opt
from metaseq_b200.tasks import LegacyTask, register_task

logger = logging.getLogger(__name__)

DEFAULT_MULTICORPUS_MAX = -1


@dataclass
class StreamingLanguageModelingConfig(MetaseqDataclass):
    data: Optional[str] = opt(None, "path to data directory with JSONL files")
    vocab_filename: Optional[str] = opt("", "path to bpe-vocab.json")
    merges_filename: Optional[str] = opt("", "path to bpe-merges.txt")
    hf_tokenizer: Optional[str] = opt("", "path to a HuggingFace tokenizers json file (alternative to vocab + merges)")
    end_of_document_symbol: Optional[str] = opt("</s>", "symbol indicating an end-of-document")
    sample_break_mode: Optional[str] = opt("none", "sample break mode: none, complete, eos_pad_8, passthrough")
    tokens_per_sample: int = opt(1024, "max number of tokens per sample for LM dataset")
    max_source_positions: Optional[int] = opt(None, "max number of tokens in the source sequence")
    max_target_positions: Optional[int] = opt(None, "max number of tokens in the target sequence")
    final_vocab_size: Optional[int] = opt(None, "force vocab size to this")
    multicorpus_sampling_alpha: Optional[float] = opt(1.0, "smoothing alpha for sample ratios across multiple datasets")
    multicorpus_sampling_maximum: Optional[float] = opt(DEFAULT_MULTICORPUS_MAX, "maximum size for example "
                                                        "proportional sampling")
    data_subshard_count: int = opt(1, "number of data subshards to use while training; subsharding allows us to "
                                   "virtually split the dataset to speed up dataset fast forwarding")
    language_modeling_type: str = opt("standard", "standard | cm3 | racm3", choices=("standard", "cm3", "racm3"))
    cm3_num_sentinel_tokens: int = opt(512, "number of special sentinel tokens to add to the vocabulary")
    cm3_lambda_sentinel_tokens: int = opt(1, "poisson rate of the number of masked spans (cm3)")
    cm3_mode: str = opt("poisson", "how to sample the number of spans", choices=("poisson", "fixed"))
    cm3_allow_across_eod_boundaries: bool = opt(True, "masked spans may cross document boundaries (the original objective); "
                                                "giving the flag turns that off")
    cm3_percent_full_document_rotation: float = opt(0.0, "fraction of documents rotated as a whole")
    num_retrieved_doc: int = opt(2, "number of retrieved documents (racm3)")
    synthetic_data: int = opt(0, "if > 0, train on this many seeded synthetic documents instead of files")
    synthetic_vocab_size: int = opt(50272, "vocabulary size of the synthetic corpus")
    synthetic_mean_doc_len: float = opt(512.0, "mean (geometric) document length of the synthetic corpus")
    add_bos_token: bool = opt(False, "prepend beginning of sentence token (<s>)")
    seed: int = opt(1, link="common.seed")
    batch_size: Optional[int] = opt(None, link="dataset.batch_size")
    batch_size_valid: Optional[int] = opt(None, link="dataset.batch_size_valid")
    update_freq: Any = opt(factory=lambda: [1], link="optimization.update_freq")


@register_task("streaming_language_modeling", dataclass=StreamingLanguageModelingConfig)
class StreamingLanguageModelingTask(LegacyTask):
    def __init__(self, args):
        super().__init__(args)
        self.tokenizer = None
        self.eod = None
        if getattr(args, "synthetic_data", 0) > 0:
            self.dictionary = Dictionary.synthetic(args.synthetic_vocab_size)
            self.eod = self.dictionary.eos()
        else:
            self._build_tokenizer_and_dictionary(args)
        final = getattr(args, "final_vocab_size", None)
        if final is not None:
            if final < len(self.dictionary):
                raise ValueError(f"incompatible: {final}, {len(self.dictionary)}")
            self.dictionary.pad_to_multiple_(final)
        else:
            self.dictionary.pad_to_multiple_(8)
        logger.info(f"dictionary: {len(self.dictionary)} types")
        self.criterion_weights = None
        self.sentinel_tokens = None

    def _build_tokenizer_and_dictionary(self, args):
        try:
            from tokenizers import ByteLevelBPETokenizer, Tokenizer
        except ImportError:
            raise ImportError("Please install huggingface/tokenizers with: pip install tokenizers")
        if getattr(args, "hf_tokenizer", ""):
            self.tokenizer = Tokenizer.from_file(args.hf_tokenizer)
        else:
            if not (os.path.exists(args.vocab_filename) and os.path.exists(args.merges_filename)):
                raise FileNotFoundError(f"cannot find {args.vocab_filename} or {args.merges_filename}; "
                                        "pass --vocab-filename and --merges-filename (or --synthetic-data N)")
            self.tokenizer = ByteLevelBPETokenizer.from_file(args.vocab_filename, args.merges_filename)
        if getattr(args, "language_modeling_type", "standard") in ("cm3", "racm3"):
            from metaseq_b200.data.cm3_dataset import sentinel_names

            self.tokenizer.add_special_tokens(sentinel_names(args.cm3_num_sentinel_tokens))
        self.dictionary = Dictionary()
        tok_vocab_size = self.tokenizer.get_vocab_size()
        for idx in range(self.dictionary.nspecial, tok_vocab_size):
            self.dictionary.add_symbol(self.tokenizer.id_to_token(idx))
        # the tokenizer's first four entries must be the dictionary specials, in this order
        for i, sym in enumerate([self.dictionary.bos_word, self.dictionary.pad_word, self.dictionary.eos_word,
                                 self.dictionary.unk_word]):
            tok = self.tokenizer.id_to_token(i)
            if tok is not None:
                assert tok == sym, f"tokenizer id {i} is {tok!r}, expected {sym!r}"
        self.eod = self.tokenizer.token_to_id(args.end_of_document_symbol)
        if self.eod is None:
            self.eod = self.dictionary.eos()

    @classmethod
    def setup_task(cls, args, **kwargs):
        return cls(args)

    # ---------------------------------------------------------------- datasets
    def _tokenize_one_json(self, json):
        text = json["text"]
        return torch.LongTensor(self.tokenizer.encode(text.rstrip()).ids + [self.eod])

    def tokenize_text(self, text: str) -> torch.Tensor:
        return torch.LongTensor(self.tokenizer.encode(text.rstrip()).ids + [self.eod])

    def _get_sample_prob(self, dataset_lens):
        prob = dataset_lens / dataset_lens.sum()
        smoothed = prob ** self.args.multicorpus_sampling_alpha
        return smoothed / smoothed.sum()

    def _alpha_sampling(self, datasets, corpora, epoch=1):
        lens = np.array([len(d) for d in datasets], dtype=float)
        logger.info(f"loaded total {lens.sum()} blocks for all corpora")
        probs = self._get_sample_prob(lens)
        size_ratio = (probs * lens.sum()) / lens
        mx = getattr(self.args, "multicorpus_sampling_maximum", DEFAULT_MULTICORPUS_MAX)
        out = []
        for i, d in enumerate(datasets):
            ratio = size_ratio[i]
            if mx != DEFAULT_MULTICORPUS_MAX and mx > 0:
                ratio = min(ratio, mx / max(1, len(d)) if len(d) * ratio > mx else ratio)
            logger.info(f"Up/Down Sampling ratio by corpus: {corpora[i]}: {ratio:0.2f}")
            out.append(ResamplingDataset(d, size_ratio=ratio, seed=self.args.seed, epoch=epoch, replace=ratio > 1.0))
        return out

    def get_shard_str(self, epoch, split):
        shards = {}
        base = os.path.join(self.args.data, split)
        for name in sorted(os.listdir(base)):
            if name.isdigit():
                shards[int(name)] = name
        assert len(shards) > 0, f"no numbered shard directories under {base}"
        order = sorted(shards)
        n_sub = max(1, int(getattr(self.args, "data_subshard_count", 1)))
        shard_idx = ((epoch - 1) // n_sub) % len(order)
        return shards[order[shard_idx]]

    def load_dataset(self, split: str, epoch=1, combine=False, **kwargs):
        """Loads one shard of ``split`` for ``epoch`` and wraps it as a block stream."""
        if getattr(self.args, "synthetic_data", 0) > 0:
            n = self.args.synthetic_data if split == "train" else max(8, self.args.synthetic_data // 16)
            dataset = SyntheticDocumentDataset(
                n, self.args.synthetic_vocab_size, self.args.synthetic_mean_doc_len,
                seed=self.args.seed + (0 if split == "train" else 7777) + 1000 * (epoch - 1), eos=self.eod)
        else:
            shard = self.get_shard_str(epoch, split)
            logger.info(f"===== Loading dataset for epoch {epoch} from shard {shard} =====")
            datasets, corpora = [], []
            sdir = os.path.join(self.args.data, split, shard)
            for fn in sorted(os.listdir(sdir)):
                if not fn.endswith(".jsonl"):
                    continue
                datasets.append(JsonlDataset(
                    path=os.path.join(sdir, fn), tokenizer=self._tokenize_one_json, epoch=epoch,
                    data_subshard_count=int(getattr(self.args, "data_subshard_count", 1)) if split == "train" else 1))
                corpora.append(os.path.splitext(fn)[0])
            assert len(datasets) > 0, f"no .jsonl files under {sdir}"
            if getattr(self.args, "multicorpus_sampling_alpha", 1.0) != 1 and split == "train":
                datasets = self._alpha_sampling(datasets, corpora, epoch)
            dataset = ConcatDataset(datasets) if len(datasets) > 1 else datasets[0]
        self.datasets[split] = DocumentToSequenceDataset(
            dataset,
            block_size=self.args.tokens_per_sample + 1,  # one extra token: input is [:-1], target [1:]
            break_mode=self.args.sample_break_mode,
            drop_last=(split == "train"),
            padding_idx=self.source_dictionary.pad(),
            seed=self.args.seed,
        )
        if getattr(self.args, "language_modeling_type", "standard") != "standard":
            from metaseq_b200.data.cm3_dataset import wrap_cm3

            self.datasets[split] = wrap_cm3(self.datasets[split], self, self.args)
        return self.datasets[split]

    def _collate_fn(self, items: List[Dict[str, Any]]):
        if len(items) > 0 and items[0] is None:
            return {}  # this rank received no data in the trailing group
        items = [x for x in items if x is not None]
        tokens = data_utils.collate_tokens([x["block"] for x in items], pad_idx=self.source_dictionary.pad(),
                                           pad_to_bsz=self.args.batch_size)
        input = tokens[:, :-1].contiguous()
        target = tokens[:, 1:].contiguous()
        ids = torch.cat([x["ids"] for x in items])
        if ids.numel() != torch.unique(ids).numel():
            n_dup = ids.numel() - torch.unique(ids).numel()
            logger.debug(f"found {n_dup}/{ids.numel()} duplicate document IDs in the same batch!")
        ntok_target = int(target.ne(self.source_dictionary.pad()).sum())
        return {
            "id": ids,
            "net_input": {"src_tokens": input},
            "target": target,
            "nsentences": input.size(0),
            "ntokens": int(input.ne(self.dictionary.pad()).sum()),
            "ntokens_target": ntok_target,
        }

    def dataset(self, split):
        return self.datasets[split]

    def get_batch_iterator(self, dataset, max_tokens=None, max_sentences=None, max_positions=None,
                           ignore_invalid_inputs=False, required_batch_size_multiple=1, seed=1, num_shards=1,
                           shard_id=0, num_workers=0, epoch=1, data_buffer_size=0, disable_iterator_cache=False,
                           batch_by_size=True, skip_remainder_batch=True):
        if not isinstance(dataset, torch.utils.data.IterableDataset):
            # a map-style dataset (the prompts of an inference request): the ordinary batch iterator
            return super().get_batch_iterator(
                dataset, max_tokens=max_tokens, max_sentences=max_sentences, max_positions=max_positions,
                ignore_invalid_inputs=ignore_invalid_inputs, required_batch_size_multiple=required_batch_size_multiple,
                seed=seed, num_shards=num_shards, shard_id=shard_id, num_workers=num_workers, epoch=epoch,
                data_buffer_size=data_buffer_size, disable_iterator_cache=disable_iterator_cache,
                batch_by_size=batch_by_size, skip_remainder_batch=skip_remainder_batch)
        assert max_tokens is None
        # larger buffer with more ranks, so that consecutive batches mix documents
        dataset.set_shuffle_buffer_size(10 * max_sentences * num_shards) if hasattr(dataset, "set_shuffle_buffer_size") \
            else None
        part = PartitionedStreamingDataset(dataset, num_shards=num_shards, shard_id=shard_id, drop_last=skip_remainder_batch)
        return iterators.StreamingEpochBatchIterator(
            dataset=part, batch_size=max_sentences, collate_fn=self._collate_fn, drop_last=skip_remainder_batch,
            num_workers=num_workers, epoch=epoch, num_shards=num_shards)

    @property
    def source_dictionary(self):
        return self.dictionary

    @property
    def target_dictionary(self):
        return self.dictionary

    def max_positions(self):
        return self.args.tokens_per_sample

    def build_dataset_for_inference(self, src_tokens, src_lengths, **kwargs):
        from metaseq_b200.tasks.language_modeling import inference_dataset

        return inference_dataset(src_tokens, src_lengths, self.source_dictionary)
