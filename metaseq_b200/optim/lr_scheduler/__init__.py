"""Learning-rate scheduler registry (``--lr-scheduler``)."""
from __future__ import annotations

from metaseq_b200 import registry

from .base_lr_scheduler import BaseLRScheduler

build_lr_scheduler_, register_lr_scheduler, LR_SCHEDULER_REGISTRY, LR_SCHEDULER_DATACLASS_REGISTRY = \
    registry.setup_registry("--lr-scheduler", base_class=BaseLRScheduler, default="fixed")


def build_lr_scheduler(cfg, optimizer):
    return build_lr_scheduler_(cfg, optimizer)


from . import cosine_lr_scheduler, fixed_schedule, inverse_square_root_schedule, polynomial_decay_schedule  # noqa: E402,F401
