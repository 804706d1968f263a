from __future__ import annotations

from metaseq_b200.dataclass.utils import gen_parser_from_dataclass
from metaseq_b200.optim.base_optimizer import BaseOptimizer


class BaseLRScheduler:
    def __init__(self, cfg, optimizer):
        if optimizer is not None and not isinstance(optimizer, BaseOptimizer):
            raise ValueError("optimizer must be an instance of BaseOptimizer")
        self.cfg = cfg
        self.optimizer = optimizer
        self.best = None

    @classmethod
    def add_args(cls, parser):
        dc = getattr(cls, "__dataclass", None)
        if dc is not None:
            gen_parser_from_dataclass(parser, dc())

    @classmethod
    def build_lr_scheduler(cls, cfg, optimizer):
        return cls(cfg, optimizer)

    def state_dict(self):
        return {"best": self.best}

    def load_state_dict(self, state_dict):
        self.best = state_dict["best"]

    def step_begin_epoch(self, epoch):
        pass

    def step(self, epoch, val_loss=None):
        if val_loss is not None:
            self.best = val_loss if self.best is None else min(self.best, val_loss)

    def step_update(self, num_updates):
        return self.optimizer.get_lr()
