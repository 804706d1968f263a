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


# Names that the reference exports at package level, resolved on first use (importing them eagerly here would pull
# the kernel loader and the parallel layers into every ``import metaseq_b200.optim``).
_LAZY = {
    "LegacyOptimizer": (".base_optimizer", "LegacyOptimizer"),
    "shard_": (".shard", "shard_"),
}


def __getattr__(name):
    try:
        module, attr = _LAZY[name]
    except KeyError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
    import importlib

    value = getattr(importlib.import_module(module, __name__), attr)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
