"""Linear warm-up from ``warmup_init_lr`` then decay proportional to 1/sqrt(update)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from metaseq_b200.dataclass.configs import MetaseqDataclass, opt

from . import register_lr_scheduler
from .base_lr_scheduler import BaseLRScheduler


@dataclass
class InverseSquareRootLRScheduleConfig(MetaseqDataclass):
    lr: Any = opt(factory=lambda: [0.25], help="learning rate (mirrors --lr)", link="optimization.lr")
    warmup_updates: int = opt(4000, "warmup the learning rate linearly for the first N updates")
    warmup_init_lr: float = opt(-1, "initial learning rate during warmup phase; default is cfg.lr")


@register_lr_scheduler("inverse_sqrt", dataclass=InverseSquareRootLRScheduleConfig)
class InverseSquareRootSchedule(BaseLRScheduler):
    def __init__(self, cfg, optimizer):
        super().__init__(cfg, optimizer)
        lr = getattr(cfg, "lr", None)
        if isinstance(lr, (list, tuple)) and len(lr) > 1:
            raise ValueError("Cannot use a fixed learning rate schedule with inverse_sqrt.")
        warmup_end_lr = lr[0] if isinstance(lr, (list, tuple)) else lr
        self.warmup_updates = max(1, int(cfg.warmup_updates))
        self.init_lr = cfg.warmup_init_lr if cfg.warmup_init_lr >= 0 else (0 if cfg.warmup_updates > 0 else warmup_end_lr)
        self.lr_step = (warmup_end_lr - self.init_lr) / self.warmup_updates
        self.decay_factor = warmup_end_lr * self.warmup_updates ** 0.5
        self.lr = self.init_lr
        self.optimizer.set_lr(self.lr)

    def step_update(self, num_updates):
        if num_updates < self.warmup_updates:
            self.lr = self.init_lr + num_updates * self.lr_step
        else:
            self.lr = self.decay_factor * num_updates ** -0.5
        self.optimizer.set_lr(self.lr)
        return self.lr
