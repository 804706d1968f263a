"""Learning-rate scheduler protocol: ``step_update`` after every optimizer update, ``step`` after every
epoch / validation, ``state_dict`` carrying the best validation loss (reference:
metaseq/optim/lr_scheduler/base_lr_scheduler.py)."""
from __future__ import annotations

from metaseq_b200.dataclass.utils import gen_parser_from_dataclass
from metaseq_b200.optim.base_optimizer import BaseOptimizer


class BaseLRScheduler:
    def __init__(self, cfg, optimizer):
        if not (optimizer is None or isinstance(optimizer, BaseOptimizer)):
            raise ValueError("optimizer must be an instance of BaseOptimizer")
        self.cfg, self.optimizer, self.best = cfg, optimizer, None

    @classmethod
    def build_lr_scheduler(cls, cfg, optimizer):
        return cls(cfg, optimizer)

    @classmethod
    def add_args(cls, parser):
        config_class = getattr(cls, "__dataclass", None)
        if config_class is not None:
            gen_parser_from_dataclass(parser, config_class())

    # ---- progress callbacks
    def step_begin_epoch(self, epoch):
        """Called before each epoch; schedulers that depend on the epoch override it."""

    def step(self, epoch, val_loss=None):
        """Called after each epoch / validation: remembers the lowest validation loss."""
        if val_loss is None:
            return
        self.best = val_loss if self.best is None else min(val_loss, self.best)

    def step_update(self, num_updates):
        """Called after each optimizer update; returns the learning rate now in effect."""
        return self.optimizer.get_lr()

    # ---- checkpointing
    def load_state_dict(self, state_dict):
        self.best = state_dict["best"]

    def state_dict(self):
        return dict(best=self.best)
