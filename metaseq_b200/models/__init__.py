"""Model and architecture registries (reference: metaseq/models/__init__.py:84-179).

``register_model(name, dataclass=...)`` registers a model class; an *architecture* is a
named function that fills default hyper-parameters on a flat namespace and maps to a
model class, selected with ``--arch``.
"""
from __future__ import annotations

import importlib
import os
from argparse import Namespace

MODEL_REGISTRY = {}
MODEL_DATACLASS_REGISTRY = {}
ARCH_MODEL_REGISTRY = {}
ARCH_MODEL_NAME_REGISTRY = {}
ARCH_MODEL_INV_REGISTRY = {}
ARCH_CONFIG_REGISTRY = {}


def build_model(cfg, task):
    """``cfg`` is the model node of the config: a flat Namespace carrying ``arch`` / ``_name``."""
    arch = getattr(cfg, "_name", None) or getattr(cfg, "arch", None)
    model_cls = ARCH_MODEL_REGISTRY.get(arch) or MODEL_REGISTRY.get(arch)
    if model_cls is None:
        raise ValueError(f"Could not infer model type from {arch!r}; known architectures: "
                         f"{sorted(ARCH_MODEL_REGISTRY)}")
    if arch in ARCH_CONFIG_REGISTRY:
        ARCH_CONFIG_REGISTRY[arch](cfg)
    return model_cls.build_model(cfg, task)


def register_model(name, dataclass=None):
    def wrap(cls):
        if name in MODEL_REGISTRY:
            raise ValueError(f"Cannot register duplicate model ({name})")
        MODEL_REGISTRY[name] = cls
        if dataclass is not None:
            cls.__dataclass = dataclass
            MODEL_DATACLASS_REGISTRY[name] = dataclass
            from metaseq_b200.dataclass.initialize import ConfigStore

            ConfigStore.instance().store(name=name, group="model", node=dataclass)
        return cls

    return wrap


def register_model_architecture(model_name, arch_name):
    def wrap(fn):
        if model_name not in MODEL_REGISTRY:
            raise ValueError(f"Cannot register model architecture for unknown model type ({model_name})")
        if arch_name in ARCH_MODEL_REGISTRY:
            raise ValueError(f"Cannot register duplicate model architecture ({arch_name})")
        if not callable(fn):
            raise ValueError(f"Model architecture must be callable ({arch_name})")
        ARCH_MODEL_REGISTRY[arch_name] = MODEL_REGISTRY[model_name]
        ARCH_MODEL_NAME_REGISTRY[arch_name] = model_name
        ARCH_MODEL_INV_REGISTRY.setdefault(model_name, []).append(arch_name)
        ARCH_CONFIG_REGISTRY[arch_name] = fn
        return fn

    return wrap


from .base_model import BaseModel, LanguageModel  # noqa: E402
from .base_decoder import BaseDecoder, IncrementalDecoder  # noqa: E402
from . import transformer_lm  # noqa: E402,F401  (registers the architectures)


# Names that the reference exports at package level, resolved on first use (importing them eagerly here would pull
# the kernel loader and the parallel layers into every ``import metaseq_b200.models``).
_LAZY = {
    "DistributedModel": (".distributed_model", "DistributedModel"),
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
