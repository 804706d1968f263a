"""Optimizer registry (``--optimizer``) and the fp16 wrappers."""
from __future__ import annotations

from metaseq_b200 import registry

from .base_optimizer import BaseOptimizer

_build_optimizer, register_optimizer, OPTIMIZER_REGISTRY, OPTIMIZER_DATACLASS_REGISTRY = registry.setup_registry(
    "--optimizer", base_class=BaseOptimizer, required=True)


def build_optimizer(cfg, params, *extra_args, **extra_kwargs):
    if all(isinstance(p, dict) for p in params):
        params = [t for p in params for t in p.values()]
    params = list(filter(lambda p: p.requires_grad, params))
    return _build_optimizer(cfg, params, *extra_args, **extra_kwargs)


from . import adam, sgd  # noqa: E402,F401
from .dynamic_loss_scaler import DynamicLossScaler  # noqa: E402,F401
from .fp16_optimizer import FP16Optimizer, MemoryEfficientFP16Optimizer  # noqa: E402,F401
