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
    lr: Any = opt(factory=lambda: [0.25], help="peak value; one entry per epoch may be given (mirrors --lr)",
                  link="optimization.lr")
    warmup_updates: int = opt(0, "updates of the linear ramp from 0 to the peak")
    zero_lr_warmup_steps: int = opt(0, "updates at exactly 0 that come before the ramp")
    force_anneal: Optional[int] = opt(None, "from this epoch on the per-epoch list is ignored")
    end_learning_rate: float = opt(0.0, "value reached at --total-num-update and held afterwards")
    power: float = opt(1.0, "exponent of the decay curve (1 = straight line)")
    total_num_update: float = opt(1000000, "update at which the decay ends")


def polynomial_lr(step: int, peak: float, floor: float, hold: int, ramp: int, end: float, power: float) -> float:
    """The schedule as a function of the update count: ``hold`` updates at 0, ``ramp`` updates of linear rise to
    ``peak``, then ``floor + (peak - floor) * (1 - progress) ** power`` until update ``end``, and ``floor`` after."""
    if hold > 0 and step <= hold:
        return 0.0
    start = hold + ramp
    if ramp > 0 and step <= start:
        return peak * (step - hold) / float(ramp)
    if step >= end:
        return floor
    left = 1 - (step - start) / (end - start)
    return floor + (peak - floor) * left ** power


@register_lr_scheduler("polynomial_decay", dataclass=PolynomialDecayLRScheduleConfig)
class PolynomialDecayLRSchedule(BaseLRScheduler):
    def __init__(self, cfg, optimizer):
        super().__init__(cfg, optimizer)
        per_epoch = list(getattr(cfg, "lr", None) or [])
        assert per_epoch, "the polynomial schedule needs --lr"
        self.lrs = per_epoch
        self.lr = per_epoch[0]
        self.zero_lr_warmup_steps = int(getattr(cfg, "zero_lr_warmup_steps", 0))
        self.warmup_updates = int(cfg.warmup_updates)
        self.end_learning_rate, self.power = cfg.end_learning_rate, cfg.power
        self.total_num_update = cfg.total_num_update
        self.force_anneal = getattr(cfg, "force_anneal", None)
        # before the first update: nothing if updates at 0 come first, else the first point of the ramp
        self.warmup_factor = 1.0 / self.warmup_updates if self.warmup_updates > 0 else 1.0
        self.optimizer.set_lr(0.0 if self.zero_lr_warmup_steps else self.warmup_factor * self.lr)

    def get_next_lr(self, epoch):
        if self.force_anneal is not None and epoch >= self.force_anneal:
            return self.optimizer.get_lr()  # keep whatever the decay has reached
        return self.lrs[min(epoch, len(self.lrs) - 1)]

    def step_begin_epoch(self, epoch):
        self.lr = self.get_next_lr(epoch)
        self.optimizer.set_lr(self.warmup_factor * self.lr)
        return self.optimizer.get_lr()

    def step_update(self, num_updates):
        in_ramp = self.zero_lr_warmup_steps < num_updates <= self.zero_lr_warmup_steps + self.warmup_updates
        if in_ramp:
            self.warmup_factor = (num_updates - self.zero_lr_warmup_steps) / float(self.warmup_updates)
        self.optimizer.set_lr(polynomial_lr(num_updates, self.lr, self.end_learning_rate, self.zero_lr_warmup_steps,
                                            self.warmup_updates, self.total_num_update, self.power))
        return self.optimizer.get_lr()
