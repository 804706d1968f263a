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
    lr: Any = opt(factory=lambda: [0.25], help="peak value when --max-lr is not given (mirrors --lr)",
                  link="optimization.lr")
    warmup_updates: int = opt(0, "updates of the linear ramp before the first cosine period")
    warmup_init_lr: float = opt(-1, "where the ramp starts (default: --min-lr)")
    min_lr: float = opt(0.0, "bottom of the first period")
    max_lr: float = opt(0.0, "top of the first period")
    t_mult: float = opt(1.0, "each period is this many times longer than the one before")
    lr_period_updates: float = opt(-1, "length of the first period in updates (default: all updates after the ramp)")
    lr_shrink: float = opt(0.1, "top and bottom are multiplied by this at every restart")
    max_update: int = opt(0, link="optimization.max_update")


def locate_period(t: float, first: float, growth: float):
    """For ``t`` updates into a train of periods of lengths ``first, first * growth, first * growth ** 2, ...``:
    ``(index of the period, its length, updates into it)``."""
    if growth == 1:
        k = math.floor(t / first)
        return k, first, t - k * first
    # the first k periods last first * (growth ** k - 1) / (growth - 1) updates in all
    k = math.floor(math.log(1 - t / first * (1 - growth), growth))
    return k, first * growth ** k, t - first * (1 - growth ** k) / (1 - growth)


@register_lr_scheduler("cosine", dataclass=CosineLRScheduleConfig)
class CosineLRSchedule(BaseLRScheduler):
    def __init__(self, cfg, optimizer):
        super().__init__(cfg, optimizer)
        given = getattr(cfg, "lr", None)
        if isinstance(given, (list, tuple)):
            if len(given) > 1:
                raise ValueError("Cannot use a fixed learning rate schedule with cosine.")
            given = given[0]
        self.min_lr = cfg.min_lr
        self.max_lr = cfg.max_lr if cfg.max_lr > 0 else given
        assert self.max_lr > self.min_lr, "max_lr must be more than min_lr"
        self.warmup_updates = int(cfg.warmup_updates)
        self.warmup_init_lr = cfg.warmup_init_lr if cfg.warmup_init_lr >= 0 else self.min_lr
        self.lr_step = (self.max_lr - self.warmup_init_lr) / self.warmup_updates if self.warmup_updates > 0 else 1
        self.t_mult, self.lr_shrink = cfg.t_mult, cfg.lr_shrink
        self.period = cfg.lr_period_updates
        if self.period <= 0:
            assert getattr(cfg, "max_update", 0) > 0, "Either --max-update or --lr-period-updates must be set"
            self.period = cfg.max_update - cfg.warmup_updates
        self.lr = self.warmup_init_lr
        self.optimizer.set_lr(self.lr)

    def step_update(self, num_updates):
        if num_updates < self.warmup_updates:
            self.lr = self.warmup_init_lr + num_updates * self.lr_step
        else:
            k, length, into = locate_period(num_updates - self.warmup_updates, self.period, self.t_mult)
            bottom, top = self.min_lr * self.lr_shrink ** k, self.max_lr * self.lr_shrink ** k
            self.lr = bottom + (top - bottom) * 0.5 * (1 + math.cos(math.pi * into / length))
        self.optimizer.set_lr(self.lr)
        return self.lr
