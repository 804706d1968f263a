"""Warm-up then polynomial decay to ``end_learning_rate`` (the OPT schedule with power 1).
Optional ``zero_lr_warmup_steps`` of exactly zero learning rate come first (reference:
metaseq/optim/lr_scheduler/polynomial_decay_schedule.py:46-104)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional

from metaseq_b200.dataclass.configs import MetaseqDataclass, opt

from . import register_lr_scheduler
from .base_lr_scheduler import BaseLRScheduler


@dataclass
class PolynomialDecayLRScheduleConfig(MetaseqDataclass):
    lr: Any = opt(factory=lambda: [0.25], help="learning rate (mirrors --lr)", link="optimization.lr")
    warmup_updates: int = opt(0, "warmup the learning rate linearly for the first N updates")
    zero_lr_warmup_steps: int = opt(0, "number of steps to run with lr = 0 in the beginning, before warmup_updates")
    force_anneal: Optional[int] = opt(None, "force annealing at specified epoch")
    end_learning_rate: float = opt(0.0, "learning rate to decay to")
    power: float = opt(1.0, "decay exponent")
    total_num_update: float = opt(1000000, "total number of updates over which to decay learning rate")


@register_lr_scheduler("polynomial_decay", dataclass=PolynomialDecayLRScheduleConfig)
class PolynomialDecayLRSchedule(BaseLRScheduler):
    def __init__(self, cfg, optimizer):
        super().__init__(cfg, optimizer)
        lr = getattr(cfg, "lr", None)
        assert lr is not None and len(lr) > 0
        self.lrs = list(lr)
        self.lr = self.lrs[0]
        self.warmup_updates = int(cfg.warmup_updates)
        self.zero_lr_warmup_steps = int(getattr(cfg, "zero_lr_warmup_steps", 0))
        self.warmup_factor = 1.0 / self.warmup_updates if self.warmup_updates > 0 else 1.0
        self.end_learning_rate = cfg.end_learning_rate
        self.total_num_update = cfg.total_num_update
        self.power = cfg.power
        self.force_anneal = getattr(cfg, "force_anneal", None)
        self.optimizer.set_lr(self.warmup_factor * self.lr if self.zero_lr_warmup_steps == 0 else 0.0)

    def get_next_lr(self, epoch):
        if self.force_anneal is None or epoch < self.force_anneal:
            return self.lrs[min(epoch, len(self.lrs) - 1)]
        return self.optimizer.get_lr()

    def step_begin_epoch(self, epoch):
        self.lr = self.get_next_lr(epoch)
        self.optimizer.set_lr(self.warmup_factor * self.lr)
        return self.optimizer.get_lr()

    def step_update(self, num_updates):
        if self.zero_lr_warmup_steps > 0 and num_updates <= self.zero_lr_warmup_steps:
            lr = 0.0
        elif self.warmup_updates > 0 and num_updates <= self.warmup_updates + self.zero_lr_warmup_steps:
            self.warmup_factor = (num_updates - self.zero_lr_warmup_steps) / float(self.warmup_updates)
            lr = self.warmup_factor * self.lr
        elif num_updates >= self.total_num_update:
            lr = self.end_learning_rate
        else:
            warm = self.warmup_updates + self.zero_lr_warmup_steps
            lr_range = self.lr - self.end_learning_rate
            remaining = 1 - (num_updates - warm) / (self.total_num_update - warm)
            lr = lr_range * remaining ** self.power + self.end_learning_rate
        self.optimizer.set_lr(lr)
        return self.optimizer.get_lr()
