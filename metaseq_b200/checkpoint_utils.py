"""Checkpoint naming, writing, discovery and loading.

On-disk contract (reference: metaseq/checkpoint_utils.py:56-81 names, :112-129 pruning,
:152-353 restore-path resolution, :372-558 shard discovery / loading, :644-684 upgrades):

    checkpoint{epoch}{suffix}.pt | checkpoint_{updates}{suffix}.pt | checkpoint_last{suffix}.pt
    suffix = "-model_part-{tp_rank}" [+ "-shard{dp_rank}" when state is sharded]

Files are ``torch.save`` pickles of plain python containers.  Writing differs from the
reference by design: the state is snapshotted to host memory by the trainer, then serialised
to ``<name>.tmp`` and atomically renamed, on a background thread when asynchronous saving is
on, so the training loop only pays for the device-to-host copy; the reference serialises
synchronously and runs only its post-save callback in a thread (metaseq/trainer.py:434-447).

Loading a sharded checkpoint onto a different data-parallel size re-slices the flat shards
(``metaseq_b200.checkpoint.flat_shards``) instead of the reference's separate merge / split
code paths (:709-906).
"""
from __future__ import annotations

import ast
import collections
import concurrent.futures
import logging
import os
import re
import shutil
import subprocess
import threading
import time
import traceback
from argparse import Namespace
from glob import glob
from typing import Any, Callable, Dict, List, Optional
from urllib.parse import urlparse

import torch

from metaseq_b200.checkpoint import flat_shards
from metaseq_b200.dataclass.utils import Cfg, overwrite_args_by_name
from metaseq_b200.file_io import PathManager, torch_load_cpu
from metaseq_b200.parallel import utils as dist_utils

logger = logging.getLogger(__name__)

_WRITER = None
_WRITER_LOCK = threading.Lock()
_PENDING: List[concurrent.futures.Future] = []


def _writer() -> concurrent.futures.ThreadPoolExecutor:
    global _WRITER
    with _WRITER_LOCK:
        if _WRITER is None:
            _WRITER = concurrent.futures.ThreadPoolExecutor(max_workers=1, thread_name_prefix="ckpt-writer")
        return _WRITER


def wait_for_pending_writes():
    """Blocks until every asynchronous checkpoint write has finished; re-raises the first error."""
    global _PENDING
    pend, _PENDING = _PENDING, []
    for f in pend:
        f.result()


class HostSnapshot:
    """Device-to-host copy of a checkpoint state that does not stall the training step.

    ``take(state)`` replaces every CUDA tensor of a nested state by a pinned host tensor filled by an asynchronous
    copy on a side stream (ordered after everything queued on the current stream so far) and returns the new state
    with an event; the host tensors are valid once ``ready()`` has returned, which the writer thread calls before
    it serialises.  The caller must keep the device tensors unchanged until the copies have run: the trainer makes
    the compute stream wait for ``event`` right before its next optimizer step, so forward and backward of that
    step overlap with the copies.  Pinned buffers are kept and reused by the next snapshot of the same layout
    (after the previous write has finished).  Host tensors in the state are cloned; on a machine without CUDA the
    snapshot is an ordinary copy.  The reference copies synchronously inside ``state_dict`` and serialises on the
    training thread (metaseq/trainer.py:410-448)."""

    def __init__(self):
        self._pool: Dict[tuple, List[torch.Tensor]] = {}
        self._stream = None
        self.event = None

    def _buffer(self, like: torch.Tensor, dtype, taken: Dict[tuple, int]) -> torch.Tensor:
        key = (tuple(like.shape), dtype)
        idx = taken.get(key, 0)
        taken[key] = idx + 1
        bucket = self._pool.setdefault(key, [])
        if idx >= len(bucket):
            bucket.append(torch.empty(like.shape, dtype=dtype, pin_memory=True))
        return bucket[idx]

    def take(self, state, cast_to_fp32: bool = False):
        from metaseq_b200 import utils

        if not torch.cuda.is_available():
            self.event = None

            def clone(t):  # a private copy: the writer thread must not see later in-place updates
                widen = cast_to_fp32 and t.dtype in (torch.float16, torch.bfloat16)
                return t.detach().to(torch.float32) if widen else t.detach().clone()

            return utils.apply_to_sample(clone, state)
        wait_for_pending_writes()  # the previous snapshot's buffers are about to be reused
        if self._stream is None:
            self._stream = torch.cuda.Stream()
        self._stream.wait_stream(torch.cuda.current_stream())
        taken: Dict[tuple, int] = {}

        def copy(t):
            dtype = torch.float32 if (cast_to_fp32 and t.dtype in (torch.float16, torch.bfloat16)) else t.dtype
            if not t.is_cuda:
                return t.detach().to(dtype).clone()
            host = self._buffer(t, dtype, taken)
            src = t.detach()
            with torch.cuda.stream(self._stream):
                host.copy_(src if src.dtype == dtype else src.to(dtype), non_blocking=True)
            src.record_stream(self._stream)
            return host

        out = utils.apply_to_sample(copy, state)
        self.event = torch.cuda.Event()
        self.event.record(self._stream)
        return out

    def ready(self):
        if self.event is not None:
            self.event.synchronize()


def _write_now(state, filename, async_callback_fn, files_to_symlink_to, ready: Optional[Callable[[], None]] = None):
    if ready is not None:
        ready()  # the host copy of the state is complete
    tmp = filename + ".tmp"
    with PathManager.open(tmp, "wb") as f:
        torch.save(state, f)
    PathManager.rename(tmp, filename)
    if async_callback_fn is not None:
        async_callback_fn(filename, files_to_symlink_to)
    elif files_to_symlink_to:
        for other in files_to_symlink_to:
            _symlink_or_copy(filename, other)


def _symlink_or_copy(src, dst):
    try:
        if os.path.lexists(dst):
            os.remove(dst)
        os.symlink(os.path.basename(src), dst)
    except OSError:
        shutil.copyfile(src, dst)


def write_checkpoint(state, filename, asynchronous=True, async_callback_fn=None, files_to_symlink_to=None,
                     ready: Optional[Callable[[], None]] = None):
    """``state`` lives in host memory, or will once ``ready()`` has returned (``HostSnapshot``)."""
    os.makedirs(os.path.dirname(os.path.abspath(filename)), exist_ok=True)
    if asynchronous:
        fut = _writer().submit(_write_now, state, filename, async_callback_fn, files_to_symlink_to, ready)
        _PENDING.append(fut)
        return fut
    _write_now(state, filename, async_callback_fn, files_to_symlink_to, ready)
    return None


# ------------------------------------------------------------------- saving
def save_checkpoint(cfg, trainer, epoch_itr, training_finished=False, async_callback_fn=None):
    """Decides which checkpoint names this update produces and has the trainer write them."""
    ckpt = cfg.checkpoint if hasattr(cfg, "checkpoint") else cfg
    if trainer.data_parallel_rank == 0:
        os.makedirs(ckpt.save_dir, exist_ok=True)
    trainer.consolidate_optimizer()
    if not trainer.should_save_checkpoint_on_current_rank:
        return
    epoch = epoch_itr.epoch
    end_of_epoch = epoch_itr.end_of_epoch()
    updates = trainer.get_num_updates()
    logger.info(f"Preparing to save checkpoint for epoch {epoch} @ {updates} updates")
    suffix = trainer.checkpoint_suffix
    conds = collections.OrderedDict()
    save_for_epoch = end_of_epoch and ckpt.save_interval_epochs > 0 and epoch % ckpt.save_interval_epochs == 0
    save_locally = ckpt.local_save_interval_updates > 0 and updates % ckpt.local_save_interval_updates == 0
    save_to_nfs = ckpt.save_interval_updates > 0 and updates % ckpt.save_interval_updates == 0
    save_for_updates = not end_of_epoch and (save_to_nfs or save_locally)
    conds[f"checkpoint{epoch}{suffix}.pt"] = save_for_epoch
    conds[f"checkpoint_{updates}{suffix}.pt"] = save_for_updates
    # every save re-points ``checkpoint_last`` (a mid-epoch one too: a restart resumes from the newest state, not
    # from the last epoch boundary); at the end of training it is written only when asked for
    # (metaseq/checkpoint_utils.py:77-81)
    conds[f"checkpoint_last{suffix}.pt"] = (training_finished and ckpt.save_last_checkpoint) or save_for_epoch \
        or save_for_updates
    extra_state = {"train_iterator": epoch_itr.state_dict()}
    names = [os.path.join(ckpt.save_dir, fn) for fn, cond in conds.items() if cond]
    if len(names) > 0:
        if PathManager.islink(names[0]):
            PathManager.rm(names[0])
        trainer.save_checkpoint(names[0], extra_state, training_finished=training_finished,
                                async_callback_fn=async_callback_fn if (save_to_nfs or training_finished) else None,
                                files_to_symlink_to=names[1:] if len(names) > 1 else None)
        logger.info(f"Saved checkpoint {names[0]} (epoch {epoch} @ {updates} updates)")
    _prune(ckpt, suffix, end_of_epoch)


def _prune(ckpt, suffix, end_of_epoch):
    if not end_of_epoch and ckpt.keep_last_updates > 0:
        for old in checkpoint_paths(ckpt.save_dir, pattern=r"checkpoint_(\d+){}\.pt".format(re.escape(suffix)))[ckpt.keep_last_updates:]:
            if os.path.lexists(old):
                os.remove(old)
    if ckpt.keep_last_epochs > 0:
        for old in checkpoint_paths(ckpt.save_dir, pattern=r"checkpoint(\d+){}\.pt".format(re.escape(suffix)))[ckpt.keep_last_epochs:]:
            if os.path.lexists(old):
                os.remove(old)


def delete_old_checkpoint_files(cfg, end_of_epoch: bool, suffix: str) -> None:
    """Keeps the newest ``keep_last_updates`` mid-epoch and ``keep_last_epochs`` end-of-epoch files of this rank's
    suffix (metaseq/checkpoint_utils.py:112-129)."""
    _prune(cfg, suffix, end_of_epoch)


def is_singleton_tensor(x: Any) -> bool:
    """A tensor without dimensions (optimizer step counts and scales are stored this way)."""
    return torch.is_tensor(x) and x.dim() == 0


def checkpoint_paths(path, pattern=r"checkpoint(\d+)\.pt"):
    """Checkpoints in ``path`` matching ``pattern``, sorted by the first group, newest first."""
    pt = re.compile(pattern)
    entries = []
    for i, f in enumerate(os.listdir(path) if os.path.isdir(path) else []):
        m = pt.fullmatch(f)
        if m is not None:
            idx = float(m.group(1)) if len(m.groups()) > 0 else i
            entries.append((idx, m.group(0)))
    return [os.path.join(path, x[1]) for x in sorted(entries, reverse=True)]


def verify_checkpoint_directory(save_dir: str) -> None:
    os.makedirs(save_dir, exist_ok=True)
    rank = dist_utils.get_global_rank()
    probe = os.path.join(save_dir, f"dummy{rank}")
    try:
        with open(probe, "w"):
            pass
    except OSError as e:
        logger.warning(f"Unable to access checkpoint save directory: {save_dir}")
        raise e
    else:
        try:
            os.remove(probe)
        except FileNotFoundError:
            pass


# ------------------------------------------------------------------ loading
def _is_checkpoint_sharded(filename: str) -> bool:
    return re.search(r"-shard\d+\.pt$", filename) is not None


def sharded_files_exist(filename: str, suffix: str) -> bool:
    return len(_shard_files_for(filename)) > 0


def _shard_files_for(filename: str) -> List[str]:
    """All ``-shardN`` siblings of ``filename`` (which may itself carry a shard number), in rank order."""
    base = re.sub(r"-shard\d+\.pt$", "", filename)
    base = re.sub(r"\.pt$", "", base)
    files = glob(base + "-shard*.pt")
    def num(p):
        m = re.search(r"-shard(\d+)\.pt$", p)
        return int(m.group(1)) if m else -1
    return sorted([f for f in files if num(f) >= 0], key=num)


def get_paths_to_load(local_path: str, suffix: str = "rank-"):
    """Shard files a rank has to read when the number of ranks differs from the number of files."""
    return _shard_files_for(local_path)


def load_checkpoint_to_cpu(path, arg_overrides=None, load_on_all_ranks=False, num_shards_expected=None,
                           shard_rank=None) -> Dict[str, Any]:
    """Loads a checkpoint into host memory.  For sharded checkpoints ``path`` names this rank's
    file; when the number of shard files on disk differs from ``num_shards_expected`` the flat
    parameters and optimizer tensors are re-sliced for ``shard_rank``."""
    files = _shard_files_for(path) if (_is_checkpoint_sharded(path) or not os.path.exists(path)) else []
    if files and num_shards_expected is not None and len(files) != num_shards_expected:
        logger.info(f"resharding {len(files)} checkpoint shards onto {num_shards_expected} data-parallel ranks")
        states = [torch_load_cpu(f) for f in files]
        state = dict(states[0])
        state["model"], state["shard_metadata"] = flat_shards.reshard_model_state(states, shard_rank, num_shards_expected)
        state["last_optimizer_state"] = flat_shards.reshard_optimizer_state(states, shard_rank, num_shards_expected)
    else:
        if not os.path.exists(path) and files:
            idx = shard_rank if shard_rank is not None and shard_rank < len(files) else 0
            path = files[idx]
        state = torch_load_cpu(path)
    if "cfg" in state and state["cfg"] is not None:
        state["cfg"] = Cfg.from_container(state["cfg"])
        if arg_overrides is not None:
            overwrite_args_by_name(state["cfg"], arg_overrides)
    elif "args" in state and state["args"] is not None and arg_overrides is not None:
        for k, v in arg_overrides.items():
            setattr(state["args"], k, v)
    return _upgrade_state_dict(state)


def _upgrade_state_dict(state):
    """Brings checkpoints written by older layouts up to the current one."""
    if "optimizer_history" not in state:
        state["optimizer_history"] = [{"criterion_name": "CrossEntropyCriterion", "best_loss": state.get("best_loss")}]
        state["last_optimizer_state"] = state.pop("optimizer", None)
    if "extra_state" not in state:
        state["extra_state"] = {"epoch": state.pop("epoch", 1), "batch_offset": state.pop("batch_offset", 0),
                                "val_loss": state.pop("val_loss", None)}
    hist = state["optimizer_history"]
    if hist and "optimizer_name" not in hist[-1]:
        hist[-1]["optimizer_name"] = "MetaseqAdam"
    if hist and "lr_scheduler_state" not in hist[-1]:
        hist[-1]["lr_scheduler_state"] = {"best": hist[-1].get("best_loss")}
    if hist and "num_updates" not in hist[-1]:
        hist[-1]["num_updates"] = 0
    if "train_iterator" not in state["extra_state"]:
        state["extra_state"]["train_iterator"] = {"epoch": state["extra_state"].get("epoch", 1),
                                                  "iterations_in_epoch": state["extra_state"].get("batch_offset", 0)}
    return state


def load_checkpoint(cfg, trainer, **passthrough_args):
    """Resolves which checkpoint to restore (explicit ``--restore-file``, ``--finetune-from-model``
    or the newest complete one in ``save_dir``), loads it and rebuilds the train iterator."""
    ckpt = cfg.checkpoint
    reset_optimizer = ckpt.reset_optimizer
    reset_lr_scheduler = ckpt.reset_lr_scheduler
    optimizer_overrides = ast.literal_eval(ckpt.optimizer_overrides)
    reset_meters = ckpt.reset_meters
    reset_dataloader = ckpt.reset_dataloader
    if ckpt.finetune_from_model is not None and (reset_optimizer or reset_lr_scheduler or reset_meters or reset_dataloader):
        raise ValueError("--finetune-from-model can not be set together with either --reset-optimizer or "
                         "reset_lr_scheduler or reset_meters or reset_dataloader")
    suffix = trainer.checkpoint_suffix
    default_restore_file = "checkpoint_last.pt"
    if ckpt.restore_file == default_restore_file:
        checkpoint_path = os.path.join(ckpt.save_dir, f"checkpoint_last{suffix}.pt")
        first_launch = not (os.path.exists(checkpoint_path) or _shard_files_for(checkpoint_path))
        if not first_launch and not os.path.exists(checkpoint_path):
            pass  # different data-parallel size than when it was written: resolved by the loader
        if first_launch:
            newest = _newest_update_checkpoint(ckpt.save_dir, suffix)
            if newest is not None:
                checkpoint_path, first_launch = newest, False
        if ckpt.finetune_from_model is not None and first_launch:
            ft = ckpt.finetune_from_model
            cand = ft.replace(".pt", suffix + ".pt") if not ft.endswith(suffix + ".pt") else ft
            if os.path.exists(cand) or _shard_files_for(cand):
                checkpoint_path = cand
            elif os.path.exists(ft):
                checkpoint_path = ft
            else:
                raise ValueError(f"--finetune-from-model {ft} does not exist")
            reset_optimizer = reset_lr_scheduler = reset_meters = reset_dataloader = True
            logger.info(f"loading pretrained model from {checkpoint_path}: optimizer, lr scheduler, meters, "
                        "dataloader will be reset")
    elif suffix is not None and suffix != "":
        # the name may be given bare ("checkpoint_3.pt") or with another rank's model-part / shard suffix
        # the parts that this rank's suffix supplies are taken off the given name first
        stem = re.sub(r"\.pt$", "", ckpt.restore_file)
        if "-shard" in suffix:
            stem = re.sub(r"-shard\d+$", "", stem)
        if "-model_part-" in suffix:
            stem = re.sub(r"-model_part-\d+$", "", stem)
        checkpoint_path = stem + suffix + ".pt"
    else:
        checkpoint_path = ckpt.restore_file
    if ckpt.restore_file != default_restore_file and ckpt.finetune_from_model:
        raise ValueError("--finetune-from-model and --restore-file (non-default value) can not be specified "
                         f"together: {cfg}")
    upload = getattr(ckpt, "cloud_upload_path", None)
    if upload and upload.startswith("nfs:"):
        # checkpoints were moved to <nfs>/checkpoint_N/checkpoint<suffix>.pt by the post-checkpoint callback:
        # a requeued job, or one with neither --restore-file nor --finetune-from-model, resumes from the newest
        # directory that holds one finished file per rank (reference: metaseq/checkpoint_utils.py:230-277)
        explicit = ckpt.restore_file != default_restore_file
        requeued = os.environ.get("SLURM_RESTART_COUNT", "0") not in ("0", "")
        if requeued or (ckpt.finetune_from_model is None and not explicit):
            latest = get_latest_complete_checkpoint_dir(upload[4:], dist_utils.get_global_world_size(), exact=True)
            checkpoint_path = os.path.join(latest, f"checkpoint{suffix}.pt") if latest else None
        elif explicit:
            checkpoint_path = ckpt.restore_file.replace(".pt", suffix + ".pt")
    requeued = os.environ.get("SLURM_RESTART_COUNT", "0") not in ("0", "")
    if upload and "blob.core.windows.net" in upload:
        # blob storage holds the checkpoints (the callback removes the local files after upload): fetch this rank's
        # file into save_dir before loading (reference: metaseq/checkpoint_utils.py:277-307, which calls a helper
        # package that is not public; here the transfers go through azcopy, as the uploads do)
        local = os.path.join(ckpt.save_dir, f"checkpoint_last{suffix}.pt")
        explicit = ckpt.restore_file != default_restore_file
        try:
            if (not explicit and ckpt.finetune_from_model is None) or requeued:
                if download_recent_ckpt(upload, local, suffix + ".pt"):
                    checkpoint_path = local
            elif explicit and "windows.net" in ckpt.restore_file:
                download_specific_ckpt(ckpt.restore_file.replace(".pt", suffix + ".pt"), local)
                checkpoint_path = local
            else:
                logger.info(f"Using checkpoint {checkpoint_path} even while uploading to blob storage")
        except FileNotFoundError:
            logger.warning("azcopy is not installed: cannot look for earlier checkpoints in blob storage; "
                           f"continuing with {checkpoint_path}")
    elif not upload and ckpt.restore_file != default_restore_file and requeued:
        # a requeued job that was started from an explicit file continues from its own newest checkpoint
        mine = os.path.join(ckpt.save_dir, f"checkpoint_last{suffix}.pt")
        if os.path.isfile(mine) or _shard_files_for(mine):
            checkpoint_path = mine
    if dist_utils.is_initialized():
        torch.distributed.barrier()
    extra_state = trainer.load_checkpoint(checkpoint_path, reset_optimizer, reset_lr_scheduler, optimizer_overrides,
                                          reset_meters=reset_meters)
    if extra_state is not None and "best" in extra_state and not reset_optimizer and not reset_meters:
        save_checkpoint.best = extra_state["best"]
    if os.environ.get("SLURM_RESTART_COUNT", "0") not in ("0", "") and extra_state is not None:
        reset_dataloader = False  # a requeued job must continue the data stream where it stopped
    if extra_state is not None and not reset_dataloader:
        itr_state = extra_state["train_iterator"]
        epoch_itr = trainer.get_train_iterator(epoch=itr_state["epoch"], **passthrough_args)
        epoch_itr.load_state_dict(itr_state)
    else:
        epoch_itr = trainer.get_train_iterator(epoch=1, **passthrough_args)
    trainer.lr_step(epoch_itr.epoch)
    return extra_state, epoch_itr


def _run_azcopy(args: List[str]):
    return subprocess.run(["azcopy", *args], stdout=subprocess.PIPE, stderr=subprocess.PIPE)


def _blob_child(url: str, name: str) -> str:
    """``url`` with ``name`` appended to its path, in front of the query (the SAS token stays last)."""
    parts = urlparse(url)
    return parts._replace(path=parts.path.rstrip("/") + "/" + name).geturl()


def download_specific_ckpt(blob_url: str, local_path: str) -> bool:
    os.makedirs(os.path.dirname(os.path.abspath(local_path)), exist_ok=True)
    res = _run_azcopy(["copy", blob_url, local_path])
    if res.returncode != 0:
        raise OSError(f"azcopy could not fetch {blob_url.split('?')[0]}: {res.stdout[-500:]!r}")
    logger.info(f"downloaded {blob_url.split('?')[0]} to {local_path}")
    return True


def download_recent_ckpt(blob_url: str, local_path: str, suffix_pt: str) -> bool:
    """Fetches ``checkpoint_<N><suffix_pt>`` with the largest N found under ``blob_url`` to ``local_path``.  Returns
    False when the container holds none (a first launch)."""
    res = _run_azcopy(["list", blob_url])
    if res.returncode != 0:
        raise OSError(f"azcopy could not list {blob_url.split('?')[0]}: {res.stdout[-500:]!r}")
    pattern = re.compile(r"(checkpoint_(\d+)" + re.escape(suffix_pt) + r")(?=[;\s]|$)")
    found = [(int(m.group(2)), m.group(1)) for m in pattern.finditer(res.stdout.decode("utf-8", "replace"))]
    if not found:
        logger.info(f"no checkpoint for this rank ({suffix_pt}) under {blob_url.split('?')[0]}")
        return False
    _, name = max(found)
    return download_specific_ckpt(_blob_child(blob_url, name), local_path)


def _newest_update_checkpoint(save_dir: str, suffix: str) -> Optional[str]:
    """Newest ``checkpoint_<updates>`` for which a file with this rank's model part exists."""
    if not os.path.isdir(save_dir):
        return None
    part = re.sub(r"-shard\d+$", "", suffix)
    best = None
    for f in os.listdir(save_dir):
        m = re.fullmatch(r"checkpoint_(\d+){}(-shard\d+)?\.pt".format(re.escape(part)), f)
        if m:
            n = int(m.group(1))
            if best is None or n > best[0]:
                best = (n, os.path.join(save_dir, f"checkpoint_{n}{suffix}.pt"))
    return best[1] if best else None


def get_latest_complete_checkpoint_dir(base: str, expected_files: int, exact: bool = False) -> Optional[str]:
    """Among ``base/checkpoint_<N>/`` directories, the largest N that holds at least (``exact``: exactly)
    ``expected_files`` finished files.  An interrupted copy leaves an incomplete directory behind, and a file
    whose name starts with ``_`` is still being copied."""
    best = None
    if not os.path.isdir(base):
        return None
    for d in os.listdir(base):
        m = re.fullmatch(r"checkpoint_(\d+)", d)
        full = os.path.join(base, d)
        if m and os.path.isdir(full):
            n_files = len([f for f in os.listdir(full) if f.endswith(".pt") and not f.startswith("_")])
            enough = n_files == expected_files if exact else n_files >= expected_files
            if not enough:
                logger.info(f"skipping checkpoint {d} because it only has {n_files} files (expected {expected_files})")
            elif best is None or int(m.group(1)) > best[0]:
                best = (int(m.group(1)), full)
    return best[1] if best else None


# ------------------------------------------------------ inference-time loading
def load_model_ensemble_and_task(filenames, arg_overrides: Optional[Dict[str, Any]] = None, task=None, strict=True,
                                 suffix="", num_shards=1, state=None, build_model_hook=None):
    """Builds the task and one model per filename from checkpoints, returning
    ``(models, cfg, task)``.  ``suffix`` is appended before ``.pt`` (model part / shard)."""
    from metaseq_b200 import tasks

    assert not (strict and num_shards > 1), "Cannot load state dict with strict=True and checkpoint shards > 1"
    ensemble = []
    cfg = None
    for filename in filenames:
        orig = filename
        assert num_shards > 0
        for shard_idx in range(num_shards):
            if num_shards == 1:
                filename = orig.replace(".pt", suffix + ".pt") if suffix and not orig.endswith(suffix + ".pt") else orig
            else:
                filename = orig[:-3] + f"_part{shard_idx}.pt"
            if not os.path.exists(filename) and not _shard_files_for(filename):
                raise IOError(f"Model file not found: {filename}")
            if state is None:
                state = load_checkpoint_to_cpu(filename, arg_overrides)
            if "cfg" in state and state["cfg"] is not None:
                cfg = state["cfg"]
            else:
                raise RuntimeError(f"Neither args nor cfg exist in state keys = {state.keys()}")
            if task is None:
                task = tasks.setup_task(cfg.task)
            if "task_state" in state:
                task.load_state_dict(state["task_state"])
            if build_model_hook is not None:
                model = build_model_hook(cfg, task)
            else:
                model = task.build_model(cfg.model)
            ms = state["model"]
            if "decoder.output_projection.weight" not in ms and "decoder.embed_tokens.weight" in ms:
                ms["decoder.output_projection.weight"] = ms["decoder.embed_tokens.weight"]
            model.load_state_dict(ms, strict=strict)
            logger.info("Done loading state dict")
            state = None
        ensemble.append(model)
    return ensemble, cfg, task
