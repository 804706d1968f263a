"""``metaseq-train``: train a model on one or more GPUs.

Flow (reference: metaseq/cli/train.py:54-224 main, :238-411 train, :427-505
validate_and_save, :535-645 post-checkpoint callback, :743-830 validate): parse flags ->
nested config -> one process per GPU -> build task, model (FSDP-wrapped when
``--ddp-backend fully_sharded``), criterion, Trainer -> restore the latest checkpoint ->
loop over epochs / updates with periodic validation and checkpointing.
"""
from __future__ import annotations

import functools
import logging
import math
import os
import re
import shutil
import socket
import subprocess
import sys
import time
from datetime import datetime, timezone
from typing import Any, Dict, List, Optional, Tuple
from urllib.parse import urlparse

import numpy as np
import torch

from metaseq_b200 import checkpoint_utils, options, tasks, utils
from metaseq_b200.data import data_utils, iterators
from metaseq_b200.dataclass.utils import Cfg, convert_namespace_to_config
from metaseq_b200.file_io import PathManager
from metaseq_b200.logging import meters, metrics, progress_bar
from metaseq_b200.ops import functional as ops_f
from metaseq_b200.parallel import utils as dist_utils
from metaseq_b200.parallel.fsdp import FullyShardedDataParallel, fsdp_enable_wrap, fsdp_wrap
from metaseq_b200.trainer import Trainer

logging.basicConfig(format="%(asctime)s | %(levelname)s | %(name)s | %(message)s", datefmt="%Y-%m-%d %H:%M:%S",
                    level=os.environ.get("LOGLEVEL", "INFO").upper(), stream=sys.stdout)
logging.Formatter.converter = time.gmtime  # UTC timestamps
logger = logging.getLogger("metaseq_b200.cli.train")


def main(cfg: Cfg) -> None:
    utils_import_user_module(cfg.common)
    ops_f.set_backend(getattr(cfg.common, "kernel_backend", "auto") or "auto")
    if getattr(cfg.common, "strict_kernels", False):
        ops_f.set_strict_kernels(True)
    if dist_utils.is_master(cfg.distributed_training) and "job_logging_cfg" in cfg:
        pass
    assert cfg.dataset.max_tokens is not None or cfg.dataset.batch_size is not None, \
        "Must specify batch size either with --max-tokens or --batch-size"
    metrics.reset()
    if cfg.common.log_file is not None:
        handler = logging.FileHandler(filename=cfg.common.log_file)
        logger.addHandler(handler)
    np.random.seed(cfg.common.seed)
    utils.set_torch_seed(cfg.common.seed)
    checkpoint_utils.verify_checkpoint_directory(cfg.checkpoint.save_dir)
    if dist_utils.is_master(cfg.distributed_training):
        logger.info(cfg.to_container() if isinstance(cfg, Cfg) else cfg)
    task = _setup_task(cfg)
    model, criterion = build_model_and_criterion(cfg, task)
    n_params = sum(p.numel() for p in model.parameters())
    logger.info(f"task: {task.__class__.__name__}; model: {model.__class__.__name__}; "
                f"criterion: {criterion.__class__.__name__}; local params: {n_params:,}")
    data_utils.raise_if_valid_subsets_unintentionally_ignored(cfg)
    if cfg.dataset.combine_valid_subsets and not cfg.dataset.disable_validation:
        task.load_dataset("valid", combine=True, epoch=1)  # valid, valid1, valid2, ... as one set
    else:
        for valid_sub_split in cfg.dataset.valid_subset.split(","):
            if valid_sub_split and not cfg.dataset.disable_validation:
                task.load_dataset(valid_sub_split, combine=False, epoch=1)
    trainer = Trainer(cfg, task, model, criterion)
    logger.info(f"training on {cfg.distributed_training.distributed_world_size} devices (GPUs/TPUs); "
                f"max tokens per GPU = {cfg.dataset.max_tokens} and batch size per GPU = {cfg.dataset.batch_size}")
    extra_state, epoch_itr = checkpoint_utils.load_checkpoint(cfg, trainer, disable_iterator_cache=True)
    max_epoch = cfg.optimization.max_epoch or math.inf
    train_meter = meters.StopwatchMeter()
    train_meter.start()
    watchdog = trainer.start_watchdog()  # None unless --watchdog-timeout is set
    try:
        while epoch_itr.next_epoch_idx <= max_epoch:
            valid_losses, should_stop = train(cfg, trainer, task, epoch_itr)
            if should_stop:
                break
            trainer.lr_step(epoch_itr.epoch, valid_losses[0] if valid_losses else None)
            epoch_itr = trainer.get_train_iterator(epoch_itr.next_epoch_idx, load_dataset=True,
                                                   disable_iterator_cache=True)
    except KeyboardInterrupt:
        if watchdog is not None and watchdog.fired:
            raise RuntimeError(f"training stopped by the watchdog: {watchdog.fired}") from None
        raise
    finally:
        if watchdog is not None:
            watchdog.stop()
    train_meter.stop()
    checkpoint_utils.wait_for_pending_writes()
    logger.info("done training in {:.1f} seconds".format(train_meter.sum))


def build_model_and_criterion(cfg, task):
    """Model wrapped per the data-parallel backend, and the criterion."""
    from metaseq_b200.parallel import symm

    symm.set_comm_backend(getattr(cfg.common, "comm_backend", "nccl"))
    if cfg.distributed_training.ddp_backend == "fully_sharded":
        extra = {"use_sharded_state": cfg.distributed_training.use_sharded_state,
                 "comm": getattr(cfg.common, "comm_backend", "nccl")}
        with fsdp_enable_wrap(cfg.distributed_training, **extra):
            model = fsdp_wrap(task.build_model(cfg.model), process_group=dist_utils.get_data_parallel_group())
    else:
        model = task.build_model(cfg.model)
    criterion = task.build_criterion(cfg.criterion)
    return model, criterion


def utils_import_user_module(common):
    if getattr(common, "user_dir", None):
        options._import_user_module(common)


def get_skip_batches(to_skip: str) -> Optional[Dict[int, int]]:
    """``"100-200,150-250"`` -> {start update: number of batches to skip}."""
    if not to_skip:
        return None
    out = {}
    for rng in to_skip.split(","):
        lo, hi = (int(x) for x in rng.split("-"))
        out[lo] = hi - lo + 1
    return out


@metrics.aggregate("train")
def train(cfg, trainer: Trainer, task, epoch_itr) -> Tuple[List[Optional[float]], bool]:
    """One epoch (or until ``max_update``)."""
    itr = epoch_itr.next_epoch_itr(fix_batches_to_gpus=cfg.distributed_training.fix_batches_to_gpus, shuffle=True)
    update_freq = cfg.optimization.update_freq[epoch_itr.epoch - 1] \
        if epoch_itr.epoch <= len(cfg.optimization.update_freq) else cfg.optimization.update_freq[-1]
    if isinstance(epoch_itr, iterators.StreamingEpochBatchIterator):
        assert update_freq == 1, "the streaming iterator yields one batch per update (--update-freq 1)"
        grouped = False
    else:
        itr = iterators.GroupedIterator(itr, update_freq, skip_remainder_batch=True)
        grouped = True
    progress = progress_bar.get_progress_bar(
        itr, log_format=cfg.common.log_format, log_file=None, log_interval=cfg.common.log_interval,
        epoch=epoch_itr.epoch,
        tensorboard_logdir=cfg.common.tensorboard_logdir if dist_utils.is_master(cfg.distributed_training) else None,
        wandb_project=cfg.common.wandb_project if dist_utils.is_master(cfg.distributed_training) else None,
        wandb_run_name=os.environ.get("WANDB_NAME", os.path.basename(cfg.checkpoint.save_dir)),
        aim_repo=cfg.common.aim_repo if dist_utils.is_master(cfg.distributed_training) else None,
        aim_run_hash=cfg.common.aim_run_hash if dist_utils.is_master(cfg.distributed_training) else None,
        aim_param_checkpoint_dir=cfg.checkpoint.save_dir)
    progress.update_config(_flatten_config(cfg))
    trainer.begin_epoch(epoch_itr.epoch)
    valid_subsets = cfg.dataset.valid_subset.split(",")
    should_stop = False
    valid_losses = [None]
    skip_batches = get_skip_batches(cfg.dataset.skip_batches)
    to_skip = 0

    def train_one(i, samples):
        with metrics.aggregate("train_inner"):
            if getattr(cfg.common, "profile", False) and trainer.get_num_updates() == 5 and \
                    dist_utils.get_global_rank() == 0:
                return _profiled_step(cfg, trainer, samples)
            return trainer.train_step(samples)

    progress_iter = iter(progress)
    i = 0
    while True:
        metrics.log_start_time("time_sample_fetch", priority=900, round=4)
        try:
            samples = next(progress_iter)
        except StopIteration:
            break
        metrics.log_stop_time("time_sample_fetch")
        if not grouped:
            samples = [samples]
        if skip_batches is not None and trainer.get_num_updates() in skip_batches and to_skip == 0:
            to_skip = skip_batches.pop(trainer.get_num_updates())
        if to_skip > 0:
            to_skip -= 1
            logger.info(f"Skipping batch at update {trainer.get_num_updates()} ({to_skip} more to skip)")
            continue
        log_output = train_one(i, samples)
        if log_output is not None:
            num_updates = trainer.get_num_updates()
            if num_updates % cfg.common.log_interval == 0:
                stats = get_training_stats(metrics.get_smoothed_values("train_inner"))
                progress.log(stats, tag="train_inner", step=num_updates)
                metrics.reset_meters("train_inner")
        end_of_epoch = not itr.has_next() if hasattr(itr, "has_next") else False
        valid_losses, should_stop = validate_and_save(cfg, trainer, task, epoch_itr, valid_subsets, end_of_epoch,
                                                      log_output is not None)
        i += 1
        if should_stop:
            break
    logger.info("end of epoch {} (average epoch stats below)".format(epoch_itr.epoch))
    stats = get_training_stats(metrics.get_smoothed_values("train"))
    progress.print(stats, tag="train", step=trainer.get_num_updates())
    metrics.reset_meters("train")
    return valid_losses, should_stop


def _profiled_step(cfg, trainer, samples):
    """Wraps one update in the torch profiler and writes a memory table and a chrome trace."""
    from torch.profiler import ProfilerActivity, profile

    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    with profile(activities=acts, profile_memory=True, with_stack=True, record_shapes=True) as prof:
        out = trainer.train_step(samples)
    sort_key = "self_cuda_memory_usage" if torch.cuda.is_available() else "self_cpu_memory_usage"
    with open(os.path.join(cfg.checkpoint.save_dir, "memory_usage.txt"), "w") as f:
        f.write(prof.key_averages(group_by_stack_n=5).table(sort_by=sort_key, row_limit=10))
    prof.export_chrome_trace(os.path.join(cfg.checkpoint.save_dir, "profiler_trace.json"))
    return out


def _flatten_config(cfg):
    out = {}
    for k, v in (cfg.items() if hasattr(cfg, "items") else []):
        if hasattr(v, "items"):
            for kk, vv in v.items():
                out[f"{k}.{kk}"] = vv
        else:
            out[k] = str(v)
    return out


def _setup_task(cfg):
    """The task; with ``--task-ddp-backend fully_sharded`` it is set up inside the sharding context, so that a model
    the task itself holds (frozen: a scorer, a teacher) is sharded too, with the settings that suit a module that is
    never updated: no fp32 master copy unless plain fp16 asks for one, fp32 gradient reduction only outside fp16
    (reference: metaseq/cli/train.py:117-136)."""
    d = cfg.distributed_training
    if getattr(d, "task_ddp_backend", "none") != "fully_sharded":
        return tasks.setup_task(cfg.task)
    saved = (d.memory_efficient_fp16, d.fp32_reduce_scatter, getattr(d, "ddp_backend", None))
    d.memory_efficient_fp16, d.fp32_reduce_scatter, d.ddp_backend = d.fp16, not d.fp16, "fully_sharded"
    try:
        with fsdp_enable_wrap(d, use_sharded_state=d.use_sharded_state):
            return tasks.setup_task(cfg.task)
    finally:
        d.memory_efficient_fp16, d.fp32_reduce_scatter, d.ddp_backend = saved


def validate_and_save(cfg, trainer: Trainer, task, epoch_itr, valid_subsets: List[str], end_of_epoch: bool,
                      was_successful_step: bool) -> Tuple[List[Optional[float]], bool]:
    num_updates = trainer.get_num_updates()
    max_update = cfg.optimization.max_update or math.inf
    should_stop = False
    if num_updates >= max_update:
        should_stop = True
        logger.info(f"Stopping training due to num_updates: {num_updates} >= max_update: {max_update}")
    save_locally = cfg.checkpoint.local_save_interval_updates > 0 and num_updates > 0 and \
        num_updates % cfg.checkpoint.local_save_interval_updates == 0
    save_to_nfs = cfg.checkpoint.save_interval_updates > 0 and num_updates > 0 and \
        num_updates % cfg.checkpoint.save_interval_updates == 0
    do_save = (end_of_epoch and cfg.checkpoint.save_interval_epochs > 0
               and epoch_itr.epoch % cfg.checkpoint.save_interval_epochs == 0) or \
              ((save_locally or save_to_nfs) and num_updates >= cfg.dataset.validate_after_updates
               and was_successful_step) or should_stop
    do_validate = (should_stop or (cfg.dataset.validate_interval_updates > 0 and num_updates > 0
                                   and num_updates % cfg.dataset.validate_interval_updates == 0
                                   and was_successful_step)) and not cfg.dataset.disable_validation \
        and num_updates >= cfg.dataset.validate_after_updates
    # save first: a crash during validation must not lose the checkpoint
    if do_save:
        checkpoint_utils.save_checkpoint(
            cfg, trainer, epoch_itr, training_finished=should_stop,
            async_callback_fn=functools.partial(post_checkpoint_callback, cfg, num_updates, should_stop)
            if cfg.checkpoint.cloud_upload_path else None)
    valid_losses = [None]
    if do_validate:
        valid_losses = validate(cfg, trainer, task, epoch_itr, valid_subsets)
    trainer.reset_dummy_batch(epoch_itr.first_batch)
    return valid_losses, should_stop


_CHECKPOINT_NAME = re.compile(r"(checkpoint(?:\d+|_\d+|_last))(.*)")


def _checkpoint_add_directory(basename):
    """``checkpoint_18-model_part-0-shard0.pt`` -> (``checkpoint_18``, ``checkpoint-model_part-0-shard0.pt``):
    on a shared file system every checkpoint gets a directory of its own and its files drop the step from their
    name, so that ``<dir>/checkpoint.pt`` is the prefix that loaders and evaluation scripts are given."""
    m = _CHECKPOINT_NAME.match(basename)
    assert m, f"checkpoint file {basename} doesn't follow the pattern {_CHECKPOINT_NAME.pattern}"
    return m.group(1), "checkpoint" + m.group(2)


def _get_basename(path):
    parsed = urlparse(path)
    return os.path.basename(parsed.path if parsed.scheme else path)


def _get_destination_path(path, destination):
    """``destination`` joined with the file name of ``path``; for a URL the name goes into the path component,
    before the query (a SAS token stays at the end)."""
    name = _get_basename(path)
    parsed = urlparse(destination)
    if parsed.scheme:
        return parsed._replace(path=os.path.join(parsed.path, name)).geturl()
    return os.path.join(destination, name)


def _copy_to_azure(source, destination, log_dir):
    stamp = datetime.now(timezone.utc).strftime("%Y-%m-%dT%H_%M_%S")
    azcopy_logs = os.path.join(log_dir, f"{_get_basename(destination)}_azcopy_logs_{stamp}")
    os.environ["AZCOPY_CONCURRENCY_VALUE"] = "10"
    os.environ["AZCOPY_LOG_LOCATION"] = azcopy_logs
    os.makedirs(azcopy_logs, exist_ok=True)
    logger.info(f"preparing to azcopy {source} to {destination}; logs in {azcopy_logs}")
    res = _run_azcopy(["azcopy", "copy", "--cap-mbps", "96.0", source, destination], stdout=subprocess.PIPE)
    if res.returncode != 0:
        print("Error: {}, azcopy failed".format(res.returncode))
        print("Azcopy stdout = {}".format(res.stdout))
        sys.exit(1)
    logger.info(f"Successfully copied {source} to {destination}")


def post_checkpoint_callback(cfg, num_updates, training_finished, filename, files_to_symlink_to):
    """Runs on the writer thread after a checkpoint file is complete (reference: metaseq/cli/train.py:535-645).

    * blob storage URL: ``azcopy`` the file to ``<url path>/<name>?<token>``, remove the local file, and copy the
      uploaded blob once more under every alias name (blob storage has no symlinks);
    * ``nfs:<dir>``: copy to ``<dir>/checkpoint_N/_checkpoint<suffix>`` and rename to ``checkpoint<suffix>`` (a
      reader never sees a partial file), remove the local file, symlink the aliases' directories' entries to it,
      then start the evaluation script if one is configured;
    * any other path: copy through the path manager, aliases as full copies;
    * no upload path: recreate the alias symlinks beside the file."""
    upload = cfg.checkpoint.cloud_upload_path
    aliases = files_to_symlink_to or []
    if upload is None:
        for other in aliases:
            if os.path.lexists(other):
                os.remove(other)
            os.symlink(os.path.basename(filename), other)
        return
    if "blob.core.windows.net" in upload:
        log_dir = os.path.dirname(filename)
        final_path = _get_destination_path(filename, upload)
        _copy_to_azure(filename, final_path, log_dir)
        if os.path.exists(filename):
            os.remove(filename)
        for other in aliases:
            _copy_to_azure(final_path, _get_destination_path(other, upload), log_dir)
    elif upload.startswith("nfs:"):
        root = upload[4:]
        checkpoint_dir, checkpoint_file = _checkpoint_add_directory(os.path.basename(filename))
        target_dir = os.path.join(root, checkpoint_dir)
        os.makedirs(target_dir, exist_ok=True)  # another worker may have made it first
        tmp_name = os.path.join(target_dir, "_" + checkpoint_file)
        final_path = os.path.join(target_dir, checkpoint_file)
        logger.info(f"Beginning copy of {filename} to NFS")
        shutil.copyfile(filename, tmp_name)
        os.replace(tmp_name, final_path)
        logger.info(f"Successfully copied {filename} to {final_path}")
        if os.path.exists(filename):
            os.remove(filename)
        for other in aliases:
            name = os.path.basename(other)
            other_dir = os.path.join(root, _checkpoint_add_directory(name)[0])
            os.makedirs(other_dir, exist_ok=True)
            dest = os.path.join(other_dir, name)
            if os.path.lexists(dest):
                os.remove(dest)
            os.symlink(final_path, dest)
        nfs_evaluation(cfg, num_updates, training_finished, checkpoint_dir, root)
    else:
        try:
            final_path = _get_destination_path(filename, upload)
            PathManager.copy_from_local(filename, final_path, overwrite=True)
            for other in aliases:
                PathManager.copy(final_path, _get_destination_path(other, upload), overwrite=True)
            if os.path.exists(filename):
                os.remove(filename)
        except (FileNotFoundError, AssertionError) as e:
            logger.info(f"could not upload {filename}: {e}")


def nfs_evaluation(cfg, num_updates, training_finished, checkpoint_dir, destination_checkpoints_dir):
    """On global rank 0, for checkpoints whose step is a multiple of ``--nfs-eval-frequency`` (and for the final
    one): wait until every rank's part has been renamed into place (names that start with ``_`` are still being
    copied), then run ``bash <script> <dir>/checkpoint.pt``.  The script path is taken relative to
    ``$METASEQ_SAVE_DIR`` when that is set (reference: metaseq/cli/train.py:648-706)."""
    ck = cfg.checkpoint
    if ck.nfs_eval_script_path is None or dist_utils.get_global_rank() != 0:
        return
    due = ck.nfs_eval_frequency > 0 and num_updates % ck.nfs_eval_frequency == 0
    if not (due or training_finished):
        return
    current = os.path.join(destination_checkpoints_dir, checkpoint_dir)
    world = cfg.distributed_training.distributed_world_size
    done = 0
    for _ in range(ck.nfs_eval_num_attempts):
        time.sleep(ck.nfs_eval_attempt_wait_minutes * 60)
        done = len([f for f in os.listdir(current) if not f.startswith("_")])
        if done == world:
            logger.info(f"All checkpoint parts for {checkpoint_dir} are in NFS, will now start to run evals")
            script = os.path.join(os.environ.get("METASEQ_SAVE_DIR", ""), ck.nfs_eval_script_path)
            res = subprocess.run(["bash", script, os.path.join(current, "checkpoint.pt")],
                                 stdout=subprocess.PIPE, stderr=subprocess.PIPE)
            if res.returncode == 0:
                logger.info(f"Successfully evaluated {checkpoint_dir}")
            else:
                logger.error(f"Error during evaluation: {res.returncode}")
                logger.error(f"Eval script stdout = {res.stdout}")
                logger.error(f"Eval script stderr = {res.stderr}")
            return
    logger.error(f"Did not evaluate {checkpoint_dir}, as only {done}/{world} checkpoint parts were copied to NFS "
                 "within waiting time")


def add_num_updates_to_stats(trainer: Trainer, stats: Dict[str, Any]) -> Dict[str, Any]:
    stats["num_updates"] = trainer.get_num_updates()
    return stats


def _run_azcopy(cmd, stdout):
    return subprocess.run(cmd, stdout=stdout)


def get_training_stats(stats: Dict[str, Any]) -> Dict[str, Any]:
    stats["wall"] = round(metrics.get_meter("default", "wall").elapsed_time, 0)
    return stats


def validate(cfg, trainer: Trainer, task, epoch_itr, subsets: List[str]) -> List[Optional[float]]:
    if cfg.dataset.fixed_validation_seed is not None:
        utils.set_torch_seed(cfg.dataset.fixed_validation_seed)
    trainer.begin_valid_epoch(epoch_itr.epoch)
    valid_losses = []
    with metrics.aggregate(new_root=True) as combined_agg:
        for subset in subsets:
            logger.info(f'begin validation on "{subset}" subset on rank {dist_utils.get_global_rank()}')
            itr = trainer.get_valid_iterator(subset).next_epoch_itr(shuffle=False, set_dataset_epoch=False)
            progress = progress_bar.get_progress_bar(
                itr, log_format=cfg.common.log_format, log_interval=cfg.common.log_interval, epoch=epoch_itr.epoch,
                prefix=f"valid on '{subset}' subset",
                tensorboard_logdir=cfg.common.tensorboard_logdir if dist_utils.is_master(cfg.distributed_training) else None,
                wandb_project=cfg.common.wandb_project if dist_utils.is_master(cfg.distributed_training) else None,
                wandb_run_name=os.environ.get("WANDB_NAME", os.path.basename(cfg.checkpoint.save_dir)),
                aim_repo=cfg.common.aim_repo if dist_utils.is_master(cfg.distributed_training) else None,
                aim_run_hash=cfg.common.aim_run_hash if dist_utils.is_master(cfg.distributed_training) else None,
                aim_param_checkpoint_dir=cfg.checkpoint.save_dir)
            with metrics.aggregate(new_root=True) as agg:
                for i, sample in enumerate(progress):
                    if cfg.dataset.max_valid_steps is not None and i > cfg.dataset.max_valid_steps:
                        break
                    trainer.valid_step(sample, num_step=i)
            stats = get_valid_stats(cfg, trainer, subset, agg.get_smoothed_values())
            progress.print(stats, tag=subset, step=trainer.get_num_updates())
            valid_losses.append(stats.get("loss"))
    stats = get_valid_stats(cfg, trainer, "combined", combined_agg.get_smoothed_values())
    return valid_losses


def get_valid_stats(cfg, trainer: Trainer, subset: str, stats: Dict[str, Any]) -> Dict[str, Any]:
    stats["num_updates"] = trainer.get_num_updates()
    return stats


def set_local_per_worker_env_variables(cfg=None):
    """Per-rank NCCL debug file and an environment dump next to the checkpoints (only when
    ``METASEQ_SAVE_DIR`` is set, as the launcher does)."""
    save_dir = os.environ.get("METASEQ_SAVE_DIR")
    if not save_dir:
        return
    os.makedirs(os.path.join(save_dir, "envs"), exist_ok=True)
    host = socket.gethostname()
    restart = os.environ.get("SLURM_RESTART_COUNT", "0")
    rank = os.environ.get("SLURM_PROCID", os.environ.get("RANK", "0"))
    os.environ.setdefault("NCCL_DEBUG_FILE", os.path.join(save_dir, f"nccl.{restart}.{host}.{rank}.%p.log"))
    with open(os.path.join(save_dir, "envs", f"env.{restart}.{host}.{rank}.txt"), "w") as f:
        for k, v in sorted(os.environ.items()):
            f.write(f"{k}={v}\n")


def cli_main(modify_parser=None, input_args=None) -> None:
    set_local_per_worker_env_variables()
    parser = options.get_training_parser()
    args = options.parse_args_and_arch(parser, input_args=input_args, modify_parser=modify_parser)
    cfg = convert_namespace_to_config(args)
    dist_utils.call_main(cfg, main)


if __name__ == "__main__":
    cli_main()
