"""Generic component registries selected by a flag (``--optimizer``,
``--lr-scheduler``, ``--criterion``, ``--bpe``, ``--tokenizer``).

Same contract as the reference (metaseq/registry.py:18-101): ``setup_registry``
returns ``(build_x, register_x, REGISTRY, DATACLASS_REGISTRY)``; a class is
registered under a name, optionally with the dataclass that declares its flags,
and ``build_x(cfg, ...)`` instantiates the class named by ``cfg._name`` (or the
flag value of a flat namespace).
"""
from __future__ import annotations

from argparse import Namespace
from typing import Any, Dict

REGISTRIES: Dict[str, Dict[str, Any]] = {}


def setup_registry(registry_name: str, base_class=None, default=None, required: bool = False):
    assert registry_name.startswith("--")
    key = registry_name[2:].replace("-", "_")
    REGISTRY: Dict[str, Any] = {}
    REGISTRY_CLASS_NAMES = set()
    DATACLASS_REGISTRY: Dict[str, Any] = {}
    if key in REGISTRIES:
        return  # registering twice would shadow earlier components
    REGISTRIES[key] = {
        "registry": REGISTRY,
        "default": default,
        "dataclass_registry": DATACLASS_REGISTRY,
        "required": required,
    }

    def build_x(cfg, *extra_args, **extra_kwargs):
        if cfg is None:
            choice = default
        elif isinstance(cfg, str):
            choice = cfg
        elif isinstance(cfg, Namespace):
            choice = getattr(cfg, "_name", None) or getattr(cfg, key, None)
        else:
            choice = cfg.get("_name") if hasattr(cfg, "get") else getattr(cfg, "_name", None)
        if choice is None:
            if required:
                raise ValueError(f"{registry_name} is required!")
            return None
        if choice not in REGISTRY:
            raise ValueError(f"unknown {registry_name} value {choice!r}; known: {sorted(REGISTRY)}")
        cls = REGISTRY[choice]
        if isinstance(cfg, str) or cfg is None:
            dc = DATACLASS_REGISTRY.get(choice)
            cfg = dc() if dc is not None else Namespace()
        builder = getattr(cls, "build_" + key, cls)
        return builder(cfg, *extra_args, **extra_kwargs)

    def register_x(name, dataclass=None):
        def wrap(cls):
            if name in REGISTRY:
                raise ValueError(f"Cannot register duplicate {key} ({name})")
            if cls.__name__ in REGISTRY_CLASS_NAMES:
                raise ValueError(f"Cannot register {key} with duplicate class name ({cls.__name__})")
            if base_class is not None and not issubclass(cls, base_class):
                raise ValueError(f"{cls.__name__} must extend {base_class.__name__}")
            if dataclass is not None:
                cls.__dataclass = dataclass
                DATACLASS_REGISTRY[name] = dataclass
                from metaseq_b200.dataclass.initialize import ConfigStore

                ConfigStore.instance().store(name=name, group=key, node=dataclass)
            REGISTRY[name] = cls
            REGISTRY_CLASS_NAMES.add(cls.__name__)
            return cls

        return wrap

    return build_x, register_x, REGISTRY, DATACLASS_REGISTRY
