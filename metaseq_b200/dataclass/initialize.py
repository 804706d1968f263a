"""Named store of configuration nodes.

The reference registers its root config, every top-level group default and every registered component's
dataclass in hydra's ``ConfigStore`` (metaseq/dataclass/initialize.py:16-27, metaseq/registry.py:91-97) so that a
config can be composed by name.  Neither hydra nor omegaconf is a dependency here: the store is a plain
process-wide table with the same calls (``instance``, ``store``, ``load``, ``list``), and ``compose`` builds a
root config from ``group=name`` choices and dotted ``key=value`` overrides.
"""
from __future__ import annotations

import copy
import dataclasses
import logging
from typing import Any, Dict, List, Optional, Sequence

logger = logging.getLogger(__name__)


class ConfigStore:
    _instance: Optional["ConfigStore"] = None

    def __init__(self):
        self._nodes: Dict[Optional[str], Dict[str, Any]] = {}

    @classmethod
    def instance(cls) -> "ConfigStore":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def store(self, name: str, node: Any, group: Optional[str] = None) -> None:
        self._nodes.setdefault(group, {})[name] = node

    def load(self, name: str, group: Optional[str] = None) -> Any:
        """A fresh instance of the stored node (a dataclass type is instantiated, an instance is copied)."""
        try:
            node = self._nodes[group][name]
        except KeyError:
            where = f"group '{group}'" if group else "the root group"
            raise KeyError(f"no config named '{name}' in {where}; known: {self.list(group)}") from None
        if isinstance(node, type):
            return node()
        return copy.deepcopy(node)

    def list(self, group: Optional[str] = None) -> List[str]:
        return sorted(self._nodes.get(group, {}))

    def groups(self) -> List[str]:
        return sorted(g for g in self._nodes if g is not None)


def hydra_init(cfg_name: str = "base_config") -> None:
    """Store the root config under ``cfg_name`` and each of its top-level groups' defaults under the group's
    field name.  Idempotent."""
    from metaseq_b200.dataclass.configs import MetaseqConfig

    cs = ConfigStore.instance()
    cs.store(name=cfg_name, node=MetaseqConfig)
    for f in dataclasses.fields(MetaseqConfig):
        if f.default_factory is not dataclasses.MISSING:
            cs.store(name=f.name, node=f.default_factory)
        else:
            cs.store(name=f.name, node=None if f.default is dataclasses.MISSING else f.default)


def _parse_scalar(text: str, like: Any) -> Any:
    if text in ("null", "None", "~"):
        return None
    if isinstance(like, bool):
        if text.lower() in ("true", "1", "yes"):
            return True
        if text.lower() in ("false", "0", "no"):
            return False
        raise ValueError(f"not a boolean: {text}")
    for cast in ((type(like),) if like is not None and not isinstance(like, (list, tuple, dict)) else ()) + (int, float):
        try:
            return cast(text)
        except (TypeError, ValueError):
            continue
    if text.lower() in ("true", "false"):
        return text.lower() == "true"
    if text.startswith("[") and text.endswith("]"):
        inner = text[1:-1].strip()
        return [_parse_scalar(t.strip(), None) for t in inner.split(",")] if inner else []
    return text


def compose(overrides: Sequence[str] = (), cfg_name: str = "base_config", deletes: Sequence[str] = ()):
    """Build a root config: ``group=name`` picks a registered component's dataclass for that group (for example
    ``task=language_modeling``), ``a.b=value`` sets one field.  Group choices apply before field overrides,
    whatever their order on the command line; groups named in ``deletes`` are set to ``None`` first.  A group
    choice that no registry knows (a bare name, as encoders without options are) is stored as that name."""
    hydra_init(cfg_name)
    import importlib

    # importing a component package registers its members (and their dataclasses) with the store
    for package in ("tasks", "models", "criterions", "optim", "optim.lr_scheduler", "data.encoders"):
        importlib.import_module("metaseq_b200." + package)
    cs = ConfigStore.instance()
    cfg = cs.load(cfg_name)
    overrides = list(overrides)
    for d in deletes:
        if hasattr(cfg, d):
            setattr(cfg, d, None)
    picks = [o for o in overrides if "." not in o.split("=", 1)[0]]
    sets = [o for o in overrides if "." in o.split("=", 1)[0]]
    for o in picks:
        key, _, value = o.partition("=")
        if not hasattr(cfg, key):
            raise KeyError(f"unknown config group '{key}'")
        if value in cs.list(key):
            node = cs.load(value, group=key)
            if hasattr(node, "_name"):
                node._name = value
            setattr(cfg, key, node)
        elif key in cs.groups():
            raise KeyError(f"no config named '{value}' in group '{key}'; known: {cs.list(key)}")
        else:
            setattr(cfg, key, value)
    for o in sets:
        path, _, value = o.partition("=")
        *parents, leaf = path.split(".")
        obj = cfg
        for p in parents:
            obj = getattr(obj, p)
            if obj is None:
                raise KeyError(f"'{p}' in '{path}' is not set; choose it first (for example {p}=<name>)")
        if not hasattr(obj, leaf):
            raise KeyError(f"unknown field '{leaf}' in '{path}'")
        setattr(obj, leaf, _parse_scalar(value, getattr(obj, leaf)))
    return cfg
