"""Task base class: owns dictionaries and datasets, builds model / criterion / generator,
and defines one training and validation step (reference: metaseq/tasks/base_task.py:47-547).
"""
from __future__ import annotations

import logging
import os
import warnings
from argparse import Namespace
from typing import Any, Callable, Dict, List

import torch

from metaseq_b200 import utils
from metaseq_b200.data import Dictionary, data_utils, iterators
from metaseq_b200.dataclass.utils import gen_parser_from_dataclass
from metaseq_b200.logging import metrics

logger = logging.getLogger(__name__)


class StatefulContainer:
    def __init__(self):
        self._state: Dict[str, Any] = {}
        self._factories: Dict[str, Callable[[], Any]] = {}

    def add_factory(self, name, factory):
        self._factories[name] = factory

    def merge_state_dict(self, state_dict):
        self._state.update(state_dict)

    @property
    def state_dict(self):
        return self._state

    def __getattr__(self, name):
        if name not in self._state and name in self._factories:
            self._state[name] = self._factories[name]()
        if name in self._state:
            return self._state[name]
        raise AttributeError(f"Task state has no factory for attribute {name}")


class BaseTask:
    @classmethod
    def add_args(cls, parser):
        dc = getattr(cls, "__dataclass", None)
        if dc is not None:
            gen_parser_from_dataclass(parser, dc())

    @staticmethod
    def logging_outputs_can_be_summed(criterion) -> bool:
        return criterion.logging_outputs_can_be_summed()

    def __init__(self, cfg, **kwargs):
        self.cfg = cfg
        self.datasets = {}
        self.dataset_to_epoch_iter = {}
        self.state = StatefulContainer()

    @classmethod
    def load_dictionary(cls, filename):
        return Dictionary.load(filename)

    @classmethod
    def build_dictionary(cls, filenames, workers=1, threshold=-1, nwords=-1, padding_factor=8):
        """A dictionary from whitespace-tokenised text files: words counted by ``workers`` processes, then cut to
        words seen at least ``threshold`` times / the ``nwords`` most frequent, padded to a multiple of
        ``padding_factor``."""
        from metaseq_b200.data.dictionary import Dictionary
        from metaseq_b200.utils import tokenize_line

        d = Dictionary()
        for filename in filenames:
            Dictionary.add_file_to_dictionary(filename, d, tokenize_line, workers)
        d.finalize(threshold=threshold, nwords=nwords, padding_factor=padding_factor)
        return d

    @classmethod
    def setup_task(cls, cfg, **kwargs):
        return cls(cfg, **kwargs)

    def has_sharded_data(self, split):
        return os.pathsep in getattr(self.cfg, "data", "")

    def load_dataset(self, split: str, combine: bool = False, task_cfg=None, **kwargs):
        raise NotImplementedError

    def dataset(self, split):
        if split not in self.datasets:
            raise KeyError("Dataset not loaded: " + split)
        return self.datasets[split]

    def filter_indices_by_size(self, indices, dataset, max_positions=None, ignore_invalid_inputs=False):
        indices, ignored = dataset.filter_indices_by_size(indices, max_positions)
        if len(ignored) > 0:
            if not ignore_invalid_inputs:
                raise Exception(f"Size of sample #{ignored[0]} is invalid (={dataset.size(ignored[0])}) since "
                                f"max_positions={max_positions}, skip this example with "
                                "--skip-invalid-size-inputs-valid-test")
            logger.warning(f"{len(ignored)} samples have invalid sizes and will be skipped, "
                           f"max_positions={max_positions}, first few sample ids={ignored[:10]}")
        return indices

    def can_reuse_epoch_itr(self, dataset):
        return getattr(dataset, "can_reuse_epoch_itr_across_epochs", False)

    def get_batch_iterator(self, dataset, max_tokens=None, max_sentences=None, max_positions=None,
                           ignore_invalid_inputs=False, required_batch_size_multiple=1, seed=1, num_shards=1,
                           shard_id=0, num_workers=0, epoch=1, data_buffer_size=0, disable_iterator_cache=False,
                           batch_by_size=True, skip_remainder_batch=False):
        """Map-style datasets: order by size, filter, bucket into batches, shard over ranks."""
        can_reuse = not disable_iterator_cache and self.can_reuse_epoch_itr(dataset)
        if can_reuse and dataset in self.dataset_to_epoch_iter:
            return self.dataset_to_epoch_iter[dataset]
        assert isinstance(dataset, torch.utils.data.Dataset)
        dataset.set_epoch(epoch)
        with utils.numpy_seed(seed):
            indices = dataset.ordered_indices()
        if max_positions is not None:
            indices = self.filter_indices_by_size(indices, dataset, max_positions, ignore_invalid_inputs)
        if batch_by_size:
            batch_sampler = dataset.batch_by_size(indices, max_tokens=max_tokens, max_sentences=max_sentences,
                                                  required_batch_size_multiple=required_batch_size_multiple)
        else:
            assert max_sentences is not None, "If batch_by_size=False, max_sentences must be passed"
            batch_sampler = list(data_utils.batch_fixed(indices, max_sentences))
        epoch_iter = iterators.EpochBatchIterator(
            dataset=dataset, collate_fn=dataset.collater, batch_sampler=batch_sampler, seed=seed,
            num_shards=num_shards, shard_id=shard_id, num_workers=num_workers, epoch=epoch,
            buffer_size=data_buffer_size, skip_remainder_batch=skip_remainder_batch)
        if can_reuse:
            self.dataset_to_epoch_iter[dataset] = epoch_iter
        return epoch_iter

    def build_model(self, cfg):
        from metaseq_b200 import models

        return models.build_model(cfg, self)

    def build_criterion(self, cfg):
        from metaseq_b200 import criterions

        return criterions.build_criterion(cfg, self)

    def build_generator(self, models, args, seq_gen_cls=None, extra_gen_cls_kwargs=None):
        from metaseq_b200.sequence_generator import SequenceGenerator

        g = lambda k, d=None: getattr(args, k, d) if not isinstance(args, dict) else args.get(k, d)
        kw = dict(
            beam_size=g("beam", 5), max_len_a=g("max_len_a", 0), max_len_b=g("max_len_b", 200),
            min_len=g("min_len", 1), temperature=g("temperature", 1.0),
            need_logprobs=g("need_logprobs", False), stop=g("stop", None),
            topp=g("sampling_topp", -1.0), profile=g("profile", False),
            omega_bound=g("omega_bound", 0.3), lambda_decay=g("lambda_decay", -1),
            alpha_presence=g("alpha_presence", 0.0), alpha_frequency=g("alpha_frequency", 0.0),
            alpha_presence_src=g("alpha_presence_src", 0.0), alpha_frequency_src=g("alpha_frequency_src", 0.0),
            alpha_src_penalty_end_idx=g("alpha_src_penalty_end_idx", -1),
        )
        kw.update(extra_gen_cls_kwargs or {})
        return (seq_gen_cls or SequenceGenerator)(models, self.target_dictionary, **kw)

    def train_step(self, sample, model, criterion, optimizer, update_num, ignore_grad=False):
        """Forward + backward of one batch; returns ``(loss, sample_size, logging_output)``."""
        model.train()
        model.set_num_updates(update_num) if hasattr(model, "set_num_updates") else None
        loss, sample_size, logging_output = criterion(model, sample)
        if ignore_grad:
            loss = loss * 0
        optimizer.backward(loss)
        return loss, sample_size, logging_output

    def valid_step(self, sample, model, criterion):
        model.eval()
        with torch.no_grad():
            loss, sample_size, logging_output = criterion(model, sample)
        return loss, sample_size, logging_output

    def optimizer_step(self, optimizer, model, update_num):
        optimizer.step()

    def inference_step(self, generator, models, sample, prefix_tokens=None, constraints=None):
        with torch.no_grad():
            return generator.generate(models, sample, prefix_tokens=prefix_tokens)

    def build_dataset_for_inference(self, src_tokens, src_lengths, **kwargs):
        raise NotImplementedError

    def get_interactive_tokens_and_lengths(self, lines, encode_fn):
        """Token tensors (and their lengths) of text lines: ``encode_fn`` (the byte-pair encoder) first, then the
        dictionary lookup without adding new symbols."""
        tokens = [self.source_dictionary.encode_line(encode_fn(line), add_if_not_exist=False).long() for line in lines]
        return tokens, [t.numel() for t in tokens]

    def begin_epoch(self, epoch, model):
        pass

    def begin_valid_epoch(self, epoch, model):
        pass

    def reduce_metrics(self, logging_outputs, criterion):
        if not any("ntokens" in log for log in logging_outputs):
            warnings.warn("ntokens not found in Criterion logging outputs, cannot log wpb or wps")
        else:
            ntokens = sum(float(log.get("ntokens", 0)) for log in logging_outputs)
            metrics.log_scalar("wpb", ntokens, priority=180, round=1)
            metrics.log_speed("wps", ntokens, priority=90, round=1)
        if not any("nsentences" in log for log in logging_outputs):
            warnings.warn("nsentences not found in Criterion logging outputs, cannot log bsz")
        else:
            nsentences = sum(float(log.get("nsentences", 0)) for log in logging_outputs)
            metrics.log_scalar("bsz", nsentences, priority=190, round=1)
        criterion.__class__.reduce_metrics(logging_outputs)

    def state_dict(self):
        return dict(self.state.state_dict) if self.state is not None else {}

    def load_state_dict(self, state_dict: Dict[str, Any]):
        if self.state is not None:
            self.state.merge_state_dict(state_dict)

    def max_positions(self):
        return None

    @property
    def source_dictionary(self):
        raise NotImplementedError

    @property
    def target_dictionary(self):
        raise NotImplementedError

    def build_tokenizer(self, args):
        from metaseq_b200.data import encoders

        return encoders.build_tokenizer(args)

    def build_bpe(self, args):
        from metaseq_b200.data import encoders

        return encoders.build_bpe(args)


class LegacyTask(BaseTask):
    """Task configured from a flat argparse namespace."""

    def __init__(self, args: Namespace):
        super().__init__(args)
        self.args = args

    @classmethod
    def setup_task(cls, args: Namespace, **kwargs):
        return cls(args, **kwargs)
