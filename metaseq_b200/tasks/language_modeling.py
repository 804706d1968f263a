"""Legacy (map-style) language-modeling task over token-block datasets.  Training normally
uses the streaming task; this one is what inference builds its batches with:
``build_dataset_for_inference`` prepends EOS to every prompt and right-pads the batch
(reference: metaseq/tasks/language_modeling.py:287-330)."""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from metaseq_b200.data import BaseDataset, Dictionary, data_utils
from metaseq_b200.dataclass.configs import MetaseqDataclass, opt
from metaseq_b200.tasks import LegacyTask, register_task

logger = logging.getLogger(__name__)


@dataclass
class LanguageModelingConfig(MetaseqDataclass):
    data: Optional[str] = opt(None, "path to data directory")
    sample_break_mode: str = opt("none", "none | complete | complete_doc | eos")
    tokens_per_sample: int = opt(1024, "max number of tokens per sample for LM dataset")
    output_dictionary_size: int = opt(-1, "limit the size of output dictionary")
    add_bos_token: bool = opt(False, "prepend beginning of sentence token (<s>)")
    max_source_positions: Optional[int] = opt(None, "max number of tokens in the source sequence")
    max_target_positions: Optional[int] = opt(None, "max number of tokens in the target sequence")
    shorten_method: str = opt("none", "none | truncate | random_crop")
    shorten_data_split_list: str = opt("", "comma-separated list of dataset splits to apply shortening to")
    vocab_filename: Optional[str] = opt("", "path to bpe-vocab.json (builds the dictionary when no dict.txt exists)")
    merges_filename: Optional[str] = opt("", "path to bpe-merges.txt")
    hf_tokenizer: Optional[str] = opt("", "path to a HuggingFace tokenizers json file (alternative to vocab + merges)")
    end_of_document_symbol: Optional[str] = opt("</s>", "symbol indicating an end-of-document")
    final_vocab_size: Optional[int] = opt(None, "force the dictionary to this size by adding padding symbols")
    pad_to_fixed_length: Optional[bool] = opt(False, "pad every batch to --tokens-per-sample")
    pad_to_fixed_bsz: Optional[bool] = opt(False, "pad every batch to the batch size with empty rows")
    shuffle_docs: bool = opt(False, "with --sample-break-mode none: shuffle whole documents before building blocks")
    batch_size: Optional[int] = opt(None, link="dataset.batch_size")
    batch_size_valid: Optional[int] = opt(None, link="dataset.batch_size_valid")
    seed: int = opt(1, link="common.seed")
    dataset_impl: Optional[str] = opt(None, link="dataset.dataset_impl")


class _PromptDataset(BaseDataset):
    """Prompts with EOS prepended; the target is the prompt shifted by one, padded at the end."""

    def __init__(self, prompts, lengths, dictionary):
        super().__init__()
        self.dictionary = dictionary
        self.items = []
        for p in prompts:
            p = torch.as_tensor(p, dtype=torch.long)
            self.items.append(torch.cat([p.new([dictionary.eos()]), p]))
        self._sizes = np.array([len(x) for x in self.items])

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        src = self.items[i]
        tgt = torch.cat([src[1:], src.new([self.dictionary.pad()])])
        return {"id": i, "source": src, "target": tgt}

    @property
    def sizes(self):
        return self._sizes

    def size(self, i):
        return int(self._sizes[i])

    def num_tokens(self, i):
        return int(self._sizes[i])

    def num_tokens_vec(self, indices):
        return self._sizes[indices]

    def ordered_indices(self):
        return np.argsort(self._sizes, kind="mergesort")

    def collater(self, samples):
        if len(samples) == 0:
            return {}
        pad = self.dictionary.pad()
        src = data_utils.collate_tokens([s["source"] for s in samples], pad)
        tgt = data_utils.collate_tokens([s["target"] for s in samples], pad)
        lengths = torch.LongTensor([s["source"].numel() for s in samples])
        return {
            "id": torch.LongTensor([s["id"] for s in samples]),
            "nsentences": len(samples),
            "ntokens": int(lengths.sum()),
            "net_input": {"src_tokens": src, "src_lengths": lengths},
            "target": tgt,
        }


def inference_dataset(src_tokens, src_lengths, dictionary):
    return _PromptDataset(src_tokens, src_lengths, dictionary)


@register_task("language_modeling", dataclass=LanguageModelingConfig)
class LanguageModelingTask(LegacyTask):
    def __init__(self, args, dictionary=None, output_dictionary=None, targets=None):
        super().__init__(args)
        self.dictionary = dictionary
        self.output_dictionary = output_dictionary or dictionary
        self.targets = targets or ["future"]

    @classmethod
    def setup_dictionary(cls, args, **kwargs):
        data = getattr(args, "data", None)
        if data:
            path = os.path.join(data.split(os.pathsep)[0], "dict.txt")
            if os.path.exists(path):
                d = Dictionary.load(path)
                logger.info(f"dictionary: {len(d)} types")
                return d, d
        vocab, merges = getattr(args, "vocab_filename", ""), getattr(args, "merges_filename", "")
        hf_file = getattr(args, "hf_tokenizer", "")
        tok = None
        if hf_file and os.path.exists(hf_file):
            from tokenizers import Tokenizer

            tok = Tokenizer.from_file(hf_file)
        elif vocab and merges and os.path.exists(vocab) and os.path.exists(merges):
            from tokenizers import ByteLevelBPETokenizer

            tok = ByteLevelBPETokenizer.from_file(vocab, merges)
        if tok is not None:
            d = Dictionary()
            for i in range(d.nspecial, tok.get_vocab_size()):
                d.add_symbol(tok.id_to_token(i))
            final = getattr(args, "final_vocab_size", None)
            if final is not None:
                if final < tok.get_vocab_size():
                    raise ValueError(f"incompatible: {final}, tok_vocab_size: {tok.get_vocab_size()}")
                d.pad_to_multiple_(final)
            else:
                d.pad_to_multiple_(8)
            return d, d
        d = Dictionary.synthetic(int(getattr(args, "synthetic_vocab_size", 50272)))
        return d, d

    @classmethod
    def setup_task(cls, args, **kwargs):
        dictionary, output_dictionary = cls.setup_dictionary(args, **kwargs)
        return cls(args, dictionary, output_dictionary)

    def load_dataset(self, split, epoch=1, combine=False, **kwargs):
        from metaseq_b200.data.data_utils import load_indexed_dataset
        from metaseq_b200.data.monolingual_dataset import MonolingualDataset
        from metaseq_b200.data.token_block_dataset import TokenBlockDataset

        paths = self.args.data.split(os.pathsep)
        data_path = paths[(epoch - 1) % len(paths)]
        dataset = load_indexed_dataset(os.path.join(data_path, split), self.dictionary,
                                       getattr(self.args, "dataset_impl", None), combine=combine)
        if dataset is None:
            raise FileNotFoundError(f"Dataset not found: {split} ({os.path.join(data_path, split)})")
        from metaseq_b200.data import data_utils as du
        from metaseq_b200.data.token_transforms import SortDataset, maybe_shorten_dataset

        dataset = maybe_shorten_dataset(dataset, split, self.args.shorten_data_split_list, self.args.shorten_method,
                                        self.args.tokens_per_sample, self.args.seed)
        common = dict(pad=self.dictionary.pad(), eos=self.dictionary.eos())
        if getattr(self.args, "shuffle_docs", False):
            assert self.args.sample_break_mode == "none", "shuffle docs is only for sample break mode none"
            docs = TokenBlockDataset(dataset, dataset.sizes, self.args.tokens_per_sample, break_mode="complete_doc",
                                     include_targets=False, **common)
            with du.numpy_seed(self.args.seed + epoch):
                order = np.random.permutation(len(docs))
            dataset = SortDataset(docs, sort_order=[order, docs.sizes])
        blocks = TokenBlockDataset(dataset, dataset.sizes, self.args.tokens_per_sample,
                                   break_mode=self.args.sample_break_mode, include_targets=True, **common)
        add_eos = self.args.sample_break_mode is not None and self.args.sample_break_mode != "none"
        fixed_len = self.args.tokens_per_sample if getattr(self.args, "pad_to_fixed_length", False) else None
        pad_bsz = None
        if getattr(self.args, "pad_to_fixed_bsz", False):
            pad_bsz = getattr(self.args, "batch_size_valid", None) if "valid" in split else getattr(self.args, "batch_size", None)
        self.datasets[split] = MonolingualDataset(
            dataset=blocks, sizes=blocks.sizes, src_vocab=self.dictionary, tgt_vocab=self.output_dictionary,
            add_eos_for_other_targets=add_eos, shuffle=True, add_bos_token=self.args.add_bos_token,
            fixed_pad_length=fixed_len, pad_to_bsz=pad_bsz)

    def build_dataset_for_inference(self, src_tokens, src_lengths, **kwargs):
        return inference_dataset(src_tokens, src_lengths, self.source_dictionary)

    def eval_lm_dataloader(self, dataset, max_tokens=36000, batch_size=None, max_positions=None, num_shards=1,
                           shard_id=0, num_workers=0, data_buffer_size=10, context_window=0):
        """Batches of ``dataset`` in corpus order for perplexity evaluation.  With ``context_window`` > 0 every
        sample is prefixed with the last ``context_window`` tokens seen so far, and the targets of that prefix are
        padding so that it is not scored twice (reference: metaseq/tasks/language_modeling.py:332-363)."""
        if context_window > 0:
            from metaseq_b200.data.lm_context_window_dataset import LMContextWindowDataset

            dataset = LMContextWindowDataset(dataset=dataset, tokens_per_sample=self.args.tokens_per_sample,
                                             context_window=context_window, pad_idx=self.source_dictionary.pad())
        epoch_itr = self.get_batch_iterator(
            dataset=dataset, max_tokens=max_tokens, max_sentences=batch_size, max_positions=max_positions,
            ignore_invalid_inputs=True, num_shards=num_shards, shard_id=shard_id, num_workers=num_workers,
            data_buffer_size=data_buffer_size, disable_iterator_cache=True)
        return epoch_itr.next_epoch_itr(shuffle=False)

    def max_positions(self):
        return getattr(self.args, "max_target_positions", None) or self.args.tokens_per_sample

    @property
    def source_dictionary(self):
        return self.dictionary

    @property
    def target_dictionary(self):
        return self.output_dictionary
