"""``metaseq-validate``: load a checkpoint and run the criterion over validation subsets
(reference: metaseq/cli/validate.py:29-144)."""
from __future__ import annotations

import ast
import logging
import os
import sys
from argparse import Namespace
from itertools import chain

import torch

from metaseq_b200 import checkpoint_utils, options, utils
from metaseq_b200.dataclass.utils import convert_namespace_to_config
from metaseq_b200.logging import metrics, progress_bar
from metaseq_b200.parallel import utils as dist_utils

logging.basicConfig(format="%(asctime)s | %(levelname)s | %(name)s | %(message)s", datefmt="%Y-%m-%d %H:%M:%S",
                    level=os.environ.get("LOGLEVEL", "INFO").upper(), stream=sys.stdout)
logger = logging.getLogger("metaseq_b200.cli.validate")


def main(cfg, override_args=None):
    if isinstance(cfg, Namespace):
        cfg = convert_namespace_to_config(cfg)
    assert cfg.dataset.max_tokens is not None or cfg.dataset.batch_size is not None, \
        "Must specify batch size either with --max-tokens or --batch-size"
    use_fp16 = cfg.common.fp16
    use_cuda = torch.cuda.is_available() and not cfg.common.cpu
    if use_cuda:
        torch.cuda.set_device(cfg.distributed_training.device_id)
    if cfg.distributed_training.distributed_world_size > 1:
        dp_world = dist_utils.get_data_parallel_world_size()
        dp_rank = dist_utils.get_data_parallel_rank()
    else:
        dp_world, dp_rank = 1, 0
    overrides = vars(override_args) if override_args is not None else {}
    overrides.update(ast.literal_eval(getattr(cfg.common_eval, "model_overrides", "{}") or "{}"))
    logger.info(f"loading model(s) from {cfg.common_eval.path}")
    models, saved_cfg, task = checkpoint_utils.load_model_ensemble_and_task(
        [cfg.common_eval.path], arg_overrides=overrides, suffix=cfg.checkpoint.checkpoint_suffix)
    model = models[0]
    for m in models:
        if use_fp16:
            m.half()
        if use_cuda:
            m.cuda()
    logger.info(saved_cfg.to_container() if hasattr(saved_cfg, "to_container") else saved_cfg)
    criterion = task.build_criterion(saved_cfg.criterion)
    criterion.eval()
    all_stats = {}
    for subset in cfg.dataset.valid_subset.split(","):
        try:
            task.load_dataset(subset, combine=False, epoch=1, task_cfg=saved_cfg.task)
            dataset = task.dataset(subset)
        except KeyError:
            raise Exception("Cannot find dataset: " + subset)
        itr = task.get_batch_iterator(
            dataset=dataset, max_tokens=cfg.dataset.max_tokens, max_sentences=cfg.dataset.batch_size,
            max_positions=utils_min(task.max_positions(), *[m.max_positions() for m in models]),
            ignore_invalid_inputs=cfg.dataset.skip_invalid_size_inputs_valid_test,
            required_batch_size_multiple=cfg.dataset.required_batch_size_multiple, seed=cfg.common.seed,
            num_shards=dp_world, shard_id=dp_rank, num_workers=cfg.dataset.num_workers,
            data_buffer_size=cfg.dataset.data_buffer_size, skip_remainder_batch=False,
        ).next_epoch_itr(shuffle=False)
        progress = progress_bar.get_progress_bar(itr, log_format=cfg.common.log_format,
                                                 log_interval=cfg.common.log_interval, prefix=f"valid on '{subset}' subset")
        log_outputs = []
        for i, sample in enumerate(progress):
            if cfg.dataset.max_valid_steps is not None and i > cfg.dataset.max_valid_steps:
                break
            if not sample:
                continue
            sample = utils.move_to_cuda(sample) if use_cuda else sample
            _loss, _sample_size, log_output = task.valid_step(sample, model, criterion)
            progress.log(log_output, step=i)
            log_outputs.append(log_output)
        if dp_world > 1:
            log_outputs = dist_utils.all_gather_list(log_outputs, max_size=cfg.common.all_gather_list_size,
                                                     group=dist_utils.get_data_parallel_group())
            log_outputs = list(chain.from_iterable(log_outputs))
        with metrics.aggregate() as agg:
            task.reduce_metrics(log_outputs, criterion)
            log_output = agg.get_smoothed_values()
        progress.print(log_output, tag=subset, step=i if log_outputs else 0)
        all_stats[subset] = log_output
    return all_stats


def utils_min(*vals):
    vals = [v for v in vals if v is not None]
    return min(vals) if vals else None


def cli_main():
    parser = options.get_validation_parser()
    args = options.parse_args_and_arch(parser)
    # only flags given explicitly override what the checkpoint stored
    override_parser = options.get_validation_parser()
    override_args = options.parse_args_and_arch(override_parser, suppress_defaults=True)
    dist_utils.call_main(convert_namespace_to_config(args), main, override_args=override_args)


if __name__ == "__main__":
    cli_main()
