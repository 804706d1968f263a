"""Constant learning rate with optional linear warm-up."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from metaseq_b200.dataclass.configs import MetaseqDataclass, opt

from . import register_lr_scheduler
from .base_lr_scheduler import BaseLRScheduler


@dataclass
class FixedLRScheduleConfig(MetaseqDataclass):
    lr: Any = opt(factory=lambda: [0.25], help="learning rate (mirrors --lr)", link="optimization.lr")
    warmup_updates: int = opt(0, "warmup the learning rate linearly for the first N updates")


@register_lr_scheduler("fixed", dataclass=FixedLRScheduleConfig)
class FixedLRSchedule(BaseLRScheduler):
    def __init__(self, cfg, optimizer):
        super().__init__(cfg, optimizer)
        lr = getattr(cfg, "lr", None)
        self.lr = lr[0] if isinstance(lr, (list, tuple)) else (lr if lr is not None else optimizer.get_lr())
        self.warmup_updates = int(getattr(cfg, "warmup_updates", 0) or 0)
        if self.warmup_updates > 0:
            self.optimizer.set_lr(self.lr / self.warmup_updates)
        else:
            self.optimizer.set_lr(self.lr)

    def step_update(self, num_updates):
        if self.warmup_updates > 0 and num_updates < self.warmup_updates:
            self.optimizer.set_lr(self.lr * (num_updates + 1) / self.warmup_updates)
        else:
            self.optimizer.set_lr(self.lr)
        return self.optimizer.get_lr()
