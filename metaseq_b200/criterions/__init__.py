"""Criterion registry (``--criterion``)."""
from __future__ import annotations

from metaseq_b200 import registry

from .base_criterion import BaseCriterion

build_criterion_, register_criterion, CRITERION_REGISTRY, CRITERION_DATACLASS_REGISTRY = registry.setup_registry(
    "--criterion", base_class=BaseCriterion, default="cross_entropy")


def build_criterion(cfg, task):
    return build_criterion_(cfg, task)


from . import cross_entropy, vocab_parallel_cross_entropy  # noqa: E402,F401
