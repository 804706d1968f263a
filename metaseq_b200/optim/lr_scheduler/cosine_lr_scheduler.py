"""Cosine annealing with warm restarts: period ``lr_period_updates`` grows by ``t_mult`` after
each restart and the peak shrinks by ``lr_shrink`` (reference:
metaseq/optim/lr_scheduler/cosine_lr_scheduler.py:116-147)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from metaseq_b200.dataclass.configs import MetaseqDataclass, opt

from . import register_lr_scheduler
from .base_lr_scheduler import BaseLRScheduler


@dataclass
class CosineLRScheduleConfig(MetaseqDataclass):
    lr: Any = opt(factory=lambda: [0.25], help="learning rate (mirrors --lr)", link="optimization.lr")
    warmup_updates: int = opt(0, "warmup the learning rate linearly for the first N updates")
    warmup_init_lr: float = opt(-1, "initial learning rate during warmup phase; default is cfg.lr")
    min_lr: float = opt(0.0, "min learning rate")
    max_lr: float = opt(0.0, "max learning rate; defaults to cfg.lr")
    t_mult: float = opt(1.0, "factor to grow the length of each period")
    lr_period_updates: float = opt(-1, "initial number of updates per period")
    lr_shrink: float = opt(0.1, "shrink factor for annealing")
    max_update: int = opt(0, link="optimization.max_update")


@register_lr_scheduler("cosine", dataclass=CosineLRScheduleConfig)
class CosineLRSchedule(BaseLRScheduler):
    def __init__(self, cfg, optimizer):
        super().__init__(cfg, optimizer)
        lr = getattr(cfg, "lr", None)
        if isinstance(lr, (list, tuple)) and len(lr) > 1:
            raise ValueError("Cannot use a fixed learning rate schedule with cosine.")
        base = lr[0] if isinstance(lr, (list, tuple)) else lr
        self.max_lr = cfg.max_lr if cfg.max_lr > 0 else base
        self.min_lr = cfg.min_lr
        assert self.max_lr > self.min_lr, "max_lr must be more than min_lr"
        warmup_end_lr = self.max_lr
        self.warmup_init_lr = cfg.warmup_init_lr if cfg.warmup_init_lr >= 0 else self.min_lr
        self.t_mult = cfg.t_mult
        self.period = cfg.lr_period_updates
        if self.period <= 0:
            assert getattr(cfg, "max_update", 0) > 0, "Either --max-update or --lr-period-updates must be set"
            self.period = cfg.max_update - cfg.warmup_updates
        self.warmup_updates = int(cfg.warmup_updates)
        self.lr_step = (warmup_end_lr - self.warmup_init_lr) / self.warmup_updates if self.warmup_updates > 0 else 1
        self.lr_shrink = cfg.lr_shrink
        self.lr = self.warmup_init_lr
        self.optimizer.set_lr(self.lr)

    def step_update(self, num_updates):
        if num_updates < self.warmup_updates:
            self.lr = self.warmup_init_lr + num_updates * self.lr_step
        else:
            curr = num_updates - self.warmup_updates
            if self.t_mult != 1:
                i = math.floor(math.log(1 - curr / self.period * (1 - self.t_mult), self.t_mult))
                t_i = self.t_mult ** i * self.period
                t_curr = curr - (1 - self.t_mult ** i) / (1 - self.t_mult) * self.period
            else:
                i = math.floor(curr / self.period)
                t_i = self.period
                t_curr = curr - self.period * i
            shrink = self.lr_shrink ** i
            lo, hi = self.min_lr * shrink, self.max_lr * shrink
            self.lr = lo + 0.5 * (hi - lo) * (1 + math.cos(math.pi * t_curr / t_i))
        self.optimizer.set_lr(self.lr)
        return self.lr
