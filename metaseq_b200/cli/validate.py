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


def _data_parallel_slot(cfg):
    """(number of data-parallel ranks, this rank's index): each rank scores its own slice of a subset."""
    if cfg.distributed_training.distributed_world_size <= 1:
        return 1, 0
    return dist_utils.get_data_parallel_world_size(), dist_utils.get_data_parallel_rank()


def _load_for_scoring(cfg, override_args, on_gpu: bool):
    """Models, the configuration stored with them, their task and an eval-mode criterion.  Flags given on this
    command line (and ``--model-overrides``) win over what the checkpoint stored."""
    overrides = dict(vars(override_args)) if override_args is not None else {}
    overrides.update(ast.literal_eval(getattr(cfg.common_eval, "model_overrides", "{}") or "{}"))
    logger.info(f"loading model(s) from {cfg.common_eval.path}")
    models, saved_cfg, task = checkpoint_utils.load_model_ensemble_and_task(
        [cfg.common_eval.path], arg_overrides=overrides, suffix=cfg.checkpoint.checkpoint_suffix)
    for m in models:
        if cfg.common.fp16:
            m.half()
        if on_gpu:
            m.cuda()
    logger.info(saved_cfg.to_container() if hasattr(saved_cfg, "to_container") else saved_cfg)
    criterion = task.build_criterion(saved_cfg.criterion)
    criterion.eval()
    return models, saved_cfg, task, criterion


def _subset_batches(cfg, task, saved_cfg, models, subset: str, dp_world: int, dp_rank: int):
    try:
        task.load_dataset(subset, combine=False, epoch=1, task_cfg=saved_cfg.task)
        dataset = task.dataset(subset)
    except KeyError:
        raise Exception("Cannot find dataset: " + subset)
    limits = [v for v in (task.max_positions(), *(m.max_positions() for m in models)) if v is not None]
    ds = cfg.dataset
    return task.get_batch_iterator(
        dataset=dataset, max_tokens=ds.max_tokens, max_sentences=ds.batch_size,
        max_positions=min(limits) if limits else None, ignore_invalid_inputs=ds.skip_invalid_size_inputs_valid_test,
        required_batch_size_multiple=ds.required_batch_size_multiple, seed=cfg.common.seed, num_shards=dp_world,
        shard_id=dp_rank, num_workers=ds.num_workers, data_buffer_size=ds.data_buffer_size,
        skip_remainder_batch=False).next_epoch_itr(shuffle=False)


def score_subset(cfg, task, model, criterion, batches, subset: str, dp_world: int, on_gpu: bool):
    """Runs the criterion over one subset and returns its aggregated statistics (summed over data-parallel ranks)."""
    bar = progress_bar.get_progress_bar(batches, log_format=cfg.common.log_format, log_interval=cfg.common.log_interval,
                                        prefix=f"valid on '{subset}' subset")
    step, per_batch = 0, []
    for step, sample in enumerate(bar):
        if cfg.dataset.max_valid_steps is not None and step > cfg.dataset.max_valid_steps:
            break
        if not sample:
            continue
        if on_gpu:
            sample = utils.move_to_cuda(sample)
        _, _, logged = task.valid_step(sample, model, criterion)
        bar.log(logged, step=step)
        per_batch.append(logged)
    if dp_world > 1:
        gathered = dist_utils.all_gather_list(per_batch, max_size=cfg.common.all_gather_list_size,
                                              group=dist_utils.get_data_parallel_group())
        per_batch = list(chain.from_iterable(gathered))
    with metrics.aggregate() as agg:
        task.reduce_metrics(per_batch, criterion)
        stats = agg.get_smoothed_values()
    bar.print(stats, tag=subset, step=step if per_batch else 0)
    return stats


def main(cfg, override_args=None):
    if isinstance(cfg, Namespace):
        cfg = convert_namespace_to_config(cfg)
    assert cfg.dataset.max_tokens is not None or cfg.dataset.batch_size is not None, \
        "Must specify batch size either with --max-tokens or --batch-size"
    on_gpu = torch.cuda.is_available() and not cfg.common.cpu
    if on_gpu:
        torch.cuda.set_device(cfg.distributed_training.device_id)
    dp_world, dp_rank = _data_parallel_slot(cfg)
    models, saved_cfg, task, criterion = _load_for_scoring(cfg, override_args, on_gpu)
    results = {}
    for subset in cfg.dataset.valid_subset.split(","):
        batches = _subset_batches(cfg, task, saved_cfg, models, subset, dp_world, dp_rank)
        results[subset] = score_subset(cfg, task, models[0], criterion, batches, subset, dp_world, on_gpu)
    return results


def cli_main():
    parser = options.get_validation_parser()
    args = options.parse_args_and_arch(parser)
    # only flags given explicitly override what the checkpoint stored
    override_parser = options.get_validation_parser()
    override_args = options.parse_args_and_arch(override_parser, suppress_defaults=True)
    dist_utils.call_main(convert_namespace_to_config(args), main, override_args=override_args)


if __name__ == "__main__":
    cli_main()
