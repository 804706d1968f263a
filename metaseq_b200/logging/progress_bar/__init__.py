"""Progress reporting sinks: JSON lines through python logging (the only ``--log-format``),
optionally mirrored to TensorBoard / Weights & Biases / Aim when those packages are present
(reference: metaseq/logging/progress_bar/)."""
from __future__ import annotations

import json
from contextlib import contextmanager
import logging
import sys
from collections import OrderedDict
from numbers import Number
from typing import Optional

import torch

from ..meters import AverageMeter, StopwatchMeter, TimeMeter

logger = logging.getLogger(__name__)


def get_progress_bar(iterator, log_format: Optional[str] = "json", log_interval: int = 100, log_file: Optional[str] = None,
                     epoch: Optional[int] = None, prefix: Optional[str] = None, tensorboard_logdir: Optional[str] = None,
                     wandb_project: Optional[str] = None, wandb_run_name: Optional[str] = None,
                     aim_repo: Optional[str] = None, aim_run_hash: Optional[str] = None, aim_param_checkpoint_dir=None):
    if log_file is not None:
        handler = logging.FileHandler(filename=log_file)
        logger.addHandler(handler)
    if log_format in (None, "json"):
        bar = JsonProgressBar(iterator, epoch, prefix, log_interval)
    elif log_format == "none":
        bar = NoopProgressBar(iterator, epoch, prefix)
    else:
        raise ValueError(f"Unknown log format: {log_format}")
    if tensorboard_logdir:
        bar = TensorboardProgressBarWrapper(bar, tensorboard_logdir)
    if wandb_project:
        bar = WandBProgressBarWrapper(bar, wandb_project, run_name=wandb_run_name)
    if aim_repo:
        bar = AimProgressBarWrapper(bar, aim_repo, aim_run_hash, aim_param_checkpoint_dir)
    return bar


def format_stat(stat):
    if isinstance(stat, Number):
        stat = "{:g}".format(stat)
    elif isinstance(stat, AverageMeter):
        stat = "{:.3f}".format(stat.avg)
    elif isinstance(stat, TimeMeter):
        stat = "{:g}".format(round(stat.avg))
    elif isinstance(stat, StopwatchMeter):
        stat = "{:g}".format(round(stat.sum))
    elif torch.is_tensor(stat):
        stat = stat.tolist()
    return stat


class BaseProgressBar:
    def __init__(self, iterable, epoch=None, prefix=None):
        self.iterable = iterable
        self.n = getattr(iterable, "n", 0)
        self.epoch = epoch
        self.prefix = ""
        if epoch is not None:
            self.prefix += "epoch {:03d}".format(epoch)
        if prefix is not None:
            self.prefix += (" | " if self.prefix != "" else "") + prefix

    def __len__(self):
        return len(self.iterable)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def __iter__(self):
        raise NotImplementedError

    def log(self, stats, tag=None, step=None):
        raise NotImplementedError

    def print(self, stats, tag=None, step=None):
        raise NotImplementedError

    def update_config(self, config):
        pass

    def _format_stats(self, stats):
        out = OrderedDict(stats)
        for k in out.keys():
            out[k] = str(format_stat(out[k]))
        return out


@contextmanager
def rename_logger(logger_, new_name):
    """Log records made inside carry ``new_name`` as their logger name (``... | train_inner | {...}``), which is
    what log scrapers key on."""
    old_name = logger_.name
    if new_name is not None:
        logger_.name = new_name
    try:
        yield logger_
    finally:
        logger_.name = old_name


class JsonProgressBar(BaseProgressBar):
    """One JSON object per ``log_interval`` steps on the python logger."""

    def __init__(self, iterable, epoch=None, prefix=None, log_interval=1000):
        super().__init__(iterable, epoch, prefix)
        self.log_interval = log_interval
        self.i = None
        self.size = None

    def __iter__(self):
        self.size = len(self.iterable)
        for i, obj in enumerate(self.iterable, start=self.n):
            self.i = i
            yield obj

    def log(self, stats, tag=None, step=None):
        step = step or self.i or 0
        if step > 0 and self.log_interval is not None and step % self.log_interval == 0:
            update = self.epoch - 1 + (self.i + 1) / float(self.size) if (self.epoch is not None and self.size) else None
            stats = self._format_stats(stats, epoch=self.epoch, update=update)
            with rename_logger(logger, tag):
                logger.info(json.dumps(stats))

    def print(self, stats, tag=None, step=None):
        self.stats = stats
        if tag is not None:
            self.stats = OrderedDict([(tag + "_" + k, v) for k, v in self.stats.items()])
        stats = self._format_stats(self.stats, epoch=self.epoch)
        with rename_logger(logger, tag):
            logger.info(json.dumps(stats))

    def _format_stats(self, stats, epoch=None, update=None):
        out = OrderedDict()
        if epoch is not None:
            out["epoch"] = epoch
        if update is not None:
            out["update"] = round(update, 3)
        for k in stats.keys():
            out[k] = format_stat(stats[k])
        return out


class NoopProgressBar(BaseProgressBar):
    def __iter__(self):
        for obj in self.iterable:
            yield obj

    def log(self, stats, tag=None, step=None):
        pass

    def print(self, stats, tag=None, step=None):
        pass


class _Wrapper(BaseProgressBar):
    def __init__(self, wrapped_bar):
        self.wrapped_bar = wrapped_bar

    def __len__(self):
        return len(self.wrapped_bar)

    def __iter__(self):
        return iter(self.wrapped_bar)

    def log(self, stats, tag=None, step=None):
        self._write(stats, tag, step)
        self.wrapped_bar.log(stats, tag=tag, step=step)

    def print(self, stats, tag=None, step=None):
        self._write(stats, tag, step)
        self.wrapped_bar.print(stats, tag=tag, step=step)

    def update_config(self, config):
        self.wrapped_bar.update_config(config)

    def _write(self, stats, tag, step):
        raise NotImplementedError


class TensorboardProgressBarWrapper(_Wrapper):
    def __init__(self, wrapped_bar, tensorboard_logdir):
        super().__init__(wrapped_bar)
        self.dir = tensorboard_logdir
        self._writers = {}
        try:
            from torch.utils.tensorboard import SummaryWriter

            self._cls = SummaryWriter
        except ImportError:
            self._cls = None
            logger.warning("tensorboard not found, please install with: pip install tensorboard")

    def _writer(self, key):
        if self._cls is None:
            return None
        if key not in self._writers:
            import os

            self._writers[key] = self._cls(os.path.join(self.dir, key))
            self._writers[key].add_text("sys.argv", " ".join(sys.argv))
        return self._writers[key]

    def _write(self, stats, tag, step):
        w = self._writer(tag or "")
        if w is None:
            return
        if step is None:
            step = stats.get("num_updates", 0)
        for k in stats.keys() - {"num_updates"}:
            v = stats[k]
            if isinstance(v, AverageMeter):
                w.add_scalar(k, v.val, step)
            elif isinstance(v, Number):
                w.add_scalar(k, v, step)
            elif torch.is_tensor(v) and v.numel() == 1:
                w.add_scalar(k, v.item(), step)
        w.flush()


class WandBProgressBarWrapper(_Wrapper):
    def __init__(self, wrapped_bar, wandb_project, run_name=None):
        super().__init__(wrapped_bar)
        try:
            import wandb

            self.wandb = wandb
            wandb.init(project=wandb_project, reinit=False, name=run_name)
        except Exception as e:
            self.wandb = None
            logger.warning(f"wandb unavailable: {e}")

    def update_config(self, config):
        if self.wandb is not None:
            self.wandb.config.update(config, allow_val_change=True)
        self.wrapped_bar.update_config(config)

    def _write(self, stats, tag, step):
        if self.wandb is None:
            return
        if step is None:
            step = stats.get("num_updates", 0)
        prefix = "" if tag is None else tag + "/"
        for k in stats.keys() - {"num_updates"}:
            v = stats[k]
            if isinstance(v, AverageMeter):
                self.wandb.log({prefix + k: v.val}, step=step)
            elif isinstance(v, Number):
                self.wandb.log({prefix + k: v}, step=step)


class AimProgressBarWrapper(_Wrapper):
    def __init__(self, wrapped_bar, aim_repo, aim_run_hash, aim_param_checkpoint_dir):
        super().__init__(wrapped_bar)
        try:
            from aim import Run

            self.run = Run(run_hash=aim_run_hash, repo=aim_repo)
        except Exception:
            self.run = None
            logger.warning("Aim not found, please install with: pip install aim")

    def _write(self, stats, tag, step):
        if self.run is None:
            return
        if step is None:
            step = stats.get("num_updates", 0)
        ctx = {"tag": tag, "subset": "train" if (tag or "").startswith("train") else "val"}
        for k in stats.keys() - {"num_updates"}:
            try:
                self.run.track(float(format_stat(stats[k])), name=k, step=step, context=ctx)
            except (TypeError, ValueError):
                pass
