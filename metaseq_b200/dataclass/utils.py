"""dataclass -> argparse flags, and flat ``Namespace`` -> nested config.

Covers what the reference does with hydra + omegaconf
(metaseq/dataclass/utils.py:55-173 ``gen_parser_from_dataclass``, :347-411
``convert_namespace_to_omegaconf``, :428-491 override helpers) without either
package: the nested config is a ``Cfg`` (a dict with attribute access) whose
``to_container()`` form is what gets pickled into checkpoints under ``cfg``.
"""
from __future__ import annotations

import argparse
import ast
import copy
import enum
import re
import typing
from argparse import ArgumentError, ArgumentParser, Namespace
from dataclasses import MISSING, fields, is_dataclass
from typing import Any, Dict, List, Optional, Tuple

from .configs import COMPONENT_GROUPS, GROUPS, MetaseqDataclass


class Cfg(dict):
    """Nested config node: a dict whose keys are also attributes."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k)

    def __setattr__(self, k, v):
        self[k] = v

    def __delattr__(self, k):
        del self[k]

    def __deepcopy__(self, memo):
        return Cfg({k: copy.deepcopy(v, memo) for k, v in self.items()})

    def get_path(self, dotted: str, default=None):
        node = self
        for part in dotted.split("."):
            if isinstance(node, Namespace):
                node = getattr(node, part, None)
            elif isinstance(node, dict) and part in node:
                node = node[part]
            else:
                return default
        return node

    def to_container(self) -> dict:
        """Plain-python copy (dicts / Namespaces / scalars) for pickling into a checkpoint."""
        out = {}
        for k, v in self.items():
            if isinstance(v, Cfg):
                out[k] = v.to_container()
            else:
                out[k] = copy.deepcopy(v)
        return out

    @staticmethod
    def from_container(d) -> "Cfg":
        if isinstance(d, Cfg):
            return d
        out = Cfg()
        for k, v in (d or {}).items():
            out[k] = Cfg.from_container(v) if isinstance(v, dict) else v
        return out


def eval_str_list(x, x_type=float):
    if x is None:
        return None
    if isinstance(x, str):
        if len(x) == 0:
            return []
        x = ast.literal_eval(x)
    try:
        return list(map(x_type, x))
    except TypeError:
        return [x_type(x)]


def eval_bool(x, default=False):
    if x is None:
        return default
    try:
        return bool(ast.literal_eval(str(x))) if not isinstance(x, bool) else x
    except (ValueError, SyntaxError):
        return default


def _strip_optional(tp):
    origin = typing.get_origin(tp)
    if origin is typing.Union:
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        if len(args) == 1:
            return args[0]
    return tp


def _flag(name: str) -> str:
    return "--" + name.replace("_", "-")


def _resolved_types(dc_cls):
    try:
        return typing.get_type_hints(dc_cls)
    except Exception:
        return {f.name: f.type for f in fields(dc_cls)}


def gen_parser_from_dataclass(parser: ArgumentParser, dataclass_instance, delete_default: bool = False,
                              with_prefix: Optional[str] = None) -> None:
    """Adds one ``--kebab-case`` flag per public field of ``dataclass_instance``.

    bool fields become ``store_true`` (``store_false`` when they default to True), list
    fields parse python-literal strings, ``choices`` / aliases / ``const`` come from the
    field metadata.  A field that mirrors another group (``link``) gets a flag only if it has a help text of its
    own (``--batch-size-valid`` mirrors ``--batch-size`` unless given); the flag then has no default, so that the
    mirrored value fills it in.  A flag that already exists on the parser is skipped, so several groups may share
    one parser.
    """
    hints = _resolved_types(type(dataclass_instance))
    for f in fields(dataclass_instance):
        linked = bool(f.metadata.get("link"))
        if f.name.startswith("_") or (linked and not f.metadata.get("help")):
            continue
        name = f.name
        flag = _flag(name) if with_prefix is None else _flag(with_prefix + "_" + name)
        tp = _strip_optional(hints.get(name, f.type))
        default = f.default if f.default is not MISSING else (
            f.default_factory() if f.default_factory is not MISSING else None)
        kwargs: Dict[str, Any] = {"help": f.metadata.get("help", "")}
        origin = typing.get_origin(tp)
        if tp is bool:
            kwargs["action"] = "store_false" if default is True else "store_true"
            kwargs["default"] = default
        elif origin in (list, List, tuple):
            inner = typing.get_args(tp)[0] if typing.get_args(tp) else str
            inner = inner if inner in (int, float, str) else str
            kwargs["type"] = (lambda s, _t=inner: eval_str_list(s, _t))
            kwargs["default"] = default
        else:
            kwargs["type"] = tp if tp in (int, float, str) else str
            kwargs["default"] = default
            if f.metadata.get("choices"):
                kwargs["choices"] = list(f.metadata["choices"])
            if f.metadata.get("argparse_const") is not None:
                kwargs["const"] = f.metadata["argparse_const"]
                kwargs["nargs"] = "?"
        if linked and tp is not bool:
            kwargs["default"] = None
        if delete_default:
            kwargs["default"] = argparse.SUPPRESS if tp is not bool else kwargs["default"]
        names = [flag]
        alias = f.metadata.get("argparse_alias")
        if alias:
            names.append(alias)
        kwargs["dest"] = name if with_prefix is None else with_prefix + "_" + name
        try:
            parser.add_argument(*names, **kwargs)
        except ArgumentError:
            pass  # already defined by another group


def populate_dataclass(dc: MetaseqDataclass, args: Namespace) -> MetaseqDataclass:
    """Copies matching attributes of a flat namespace onto a dataclass instance."""
    for name in dc.field_names():
        if hasattr(args, name):
            setattr(dc, name, getattr(args, name))
    return dc


def _component_node(args: Namespace, group: str):
    """Config node of one registry component (model, task, criterion, ...).

    A component registered with a dataclass gets that dataclass filled from the flat
    namespace; one registered without (e.g. the model, whose flags are added by
    ``add_args`` and completed by the architecture function) keeps the whole flat
    namespace, which is how the model sees flags such as ``sequence_parallel``."""
    from metaseq_b200 import registry as _registry

    if group == "model":
        arch = getattr(args, "arch", None)
        if arch is None:
            return None
        ns = Namespace(**vars(args))
        ns._name = arch
        return ns
    if group == "task":
        from metaseq_b200.tasks import TASK_DATACLASS_REGISTRY

        name = getattr(args, "task", None)
        reg = TASK_DATACLASS_REGISTRY
    else:
        flag = group  # registries are keyed by their flag name
        name = getattr(args, flag, None)
        reg = _registry.REGISTRIES.get(flag, {}).get("dataclass_registry", {})
    if name is None:
        return None
    dc_cls = reg.get(name)
    if dc_cls is None:
        ns = Namespace(**vars(args))
        ns._name = name
        return ns
    dc = populate_dataclass(dc_cls(), args)
    node = Cfg(dc.to_dict())
    node["_name"] = name
    return node


def _apply_links(cfg: Cfg):
    for gname, gcls in GROUPS.items():
        for f in fields(gcls):
            link = f.metadata.get("link")
            if not link:
                continue
            src = cfg.get_path(link)
            cur = cfg[gname].get(f.name)
            default = f.default if f.default is not MISSING else None
            if cur is None or cur == default:
                cfg[gname][f.name] = src


def convert_namespace_to_config(args: Namespace) -> Cfg:
    """Flat argparse namespace -> nested ``Cfg`` with the reference's group layout
    (common / distributed_training / dataset / optimization / checkpoint / generation /
    eval_lm / reshard / ema + model / task / criterion / optimizer / lr_scheduler / bpe)."""
    cfg = Cfg()
    for gname, gcls in GROUPS.items():
        cfg[gname] = Cfg(populate_dataclass(gcls(), args).to_dict())
    if getattr(args, "memory_efficient_fp16", False):
        cfg.common.fp16 = True
    _apply_links(cfg)
    for group in COMPONENT_GROUPS:
        try:
            cfg[group] = _component_node(args, group)
        except ImportError:
            cfg[group] = None
    # the checkpoint group carries the flags that wrap the model
    return cfg


def config_to_namespace(cfg: Cfg) -> Namespace:
    """Best-effort inverse of ``convert_namespace_to_config`` (used by tools that only have a
    checkpoint's ``cfg``)."""
    ns = Namespace()
    for gname in GROUPS:
        for k, v in (cfg.get(gname) or {}).items():
            setattr(ns, k, v)
    for group in COMPONENT_GROUPS:
        node = cfg.get(group)
        if node is None:
            continue
        items = vars(node).items() if isinstance(node, Namespace) else node.items()
        for k, v in items:
            if k == "_name":
                setattr(ns, "arch" if group == "model" else group, v)
            elif not hasattr(ns, k):
                setattr(ns, k, v)
    return ns


def overwrite_args_by_name(cfg, overrides: Dict[str, Any]):
    """Sets every key of ``overrides`` wherever it occurs in the config tree
    (``--model-overrides`` / ``--optimizer-overrides`` applied onto a checkpoint's cfg)."""
    if isinstance(cfg, Namespace):
        for k, v in overrides.items():
            if hasattr(cfg, k):
                setattr(cfg, k, v)
        return cfg
    for k in list(cfg.keys()):
        v = cfg[k]
        if isinstance(v, (dict, Namespace)):
            overwrite_args_by_name(v, overrides)
        elif k in overrides:
            cfg[k] = overrides[k]
    for k, v in overrides.items():
        if isinstance(v, dict) and k in cfg and isinstance(cfg[k], dict):
            cfg[k].update(v)
    return cfg


def interpret_dc_type(field_type):
    """The type an ``argparse`` argument should parse: ``Optional[T]`` -> ``T``, ``Any`` -> ``str``."""
    if isinstance(field_type, str):
        raise RuntimeError("field should be a type")
    if field_type is Any:
        return str
    return _strip_optional(field_type)


def _override_value(v) -> str:
    if v is None:
        return "null"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (list, tuple)):
        return "[" + ",".join(_override_value(x) for x in v) + "]"
    if isinstance(v, enum.Enum):
        return str(v.value)
    return str(v)


def _override_attr(prefix: str, dc_cls, args: Namespace) -> List[str]:
    """``prefix.field=value`` for every field of ``dc_cls`` that ``args`` carries."""
    out = []
    for f in fields(dc_cls):
        if f.name != "_name" and hasattr(args, f.name):
            out.append(f"{prefix}.{f.name}={_override_value(getattr(args, f.name))}")
    return out


def migrate_registry(name, value, registry, args, overrides, deletes, use_name_as_val=False):
    """One component group of a flat namespace as overrides: a registered choice with a dataclass becomes
    ``group=choice``, ``group._name=choice`` and its fields; a bare name is kept if ``use_name_as_val``; anything
    else puts the group on the delete list."""
    if value in registry:
        overrides.append(f"{name}={value}")
        overrides.append(f"{name}._name={value}")
        overrides.extend(_override_attr(name, registry[value], args))
    elif use_name_as_val and value is not None:
        overrides.append(f"{name}={value}")
    else:
        deletes.append(name)


def override_module_args(args: Namespace) -> Tuple[List[str], List[str]]:
    """A flat namespace as ``(overrides, deletes)``: ``key=value`` strings that ``dataclass.initialize.compose``
    applies to the root config, and the component groups that the namespace does not select (reference:
    metaseq/dataclass/utils.py:287-345)."""
    overrides: List[str] = []
    deletes: List[str] = []
    for gname, gcls in GROUPS.items():
        overrides.extend(_override_attr(gname, gcls, args))
    if args is None:
        return overrides, deletes
    if hasattr(args, "task"):
        from metaseq_b200.tasks import TASK_DATACLASS_REGISTRY

        migrate_registry("task", args.task, TASK_DATACLASS_REGISTRY, args, overrides, deletes)
    else:
        deletes.append("task")
    from metaseq_b200.registry import REGISTRIES

    core = {"criterion", "optimizer", "lr_scheduler"}
    for key, reg in REGISTRIES.items():
        if hasattr(args, key):
            migrate_registry(key, getattr(args, key), reg["dataclass_registry"], args, overrides, deletes,
                             use_name_as_val=key not in core)
        else:
            deletes.append(key)
    from metaseq_b200.models import ARCH_MODEL_NAME_REGISTRY, ARCH_MODEL_REGISTRY, MODEL_DATACLASS_REGISTRY

    arch = getattr(args, "arch", None)
    dc = MODEL_DATACLASS_REGISTRY.get(ARCH_MODEL_NAME_REGISTRY.get(arch)) if arch in ARCH_MODEL_REGISTRY else None
    if dc is not None:
        overrides.append(f"model={ARCH_MODEL_NAME_REGISTRY[arch]}")
        overrides.append(f"model._name={arch}")
        overrides.extend(_override_attr("model", dc, args))
    else:
        deletes.append("model")
    return overrides, deletes


def get(cfg_or_ns, key: str, default=None):
    """Attribute/key lookup that works on ``Cfg``, dicts and Namespaces."""
    if cfg_or_ns is None:
        return default
    if isinstance(cfg_or_ns, dict):
        return cfg_or_ns.get(key, default)
    return getattr(cfg_or_ns, key, default)


# ------------------------------------------------------------ names of the reference's config helpers
convert_namespace_to_omegaconf = convert_namespace_to_config  # the config tree here is a plain ``Cfg``, not OmegaConf


def overwrite_keys_not_present(cfg, overrides: Dict[str, Any]):
    """For two-level ``{group: {key: value}}`` overrides: adds the keys that a checkpoint's group does not have yet
    (options introduced after it was written) and leaves existing ones alone (metaseq/dataclass/utils.py:480-491)."""
    for group, leaves in overrides.items():
        if group in cfg and isinstance(leaves, dict) and isinstance(cfg[group], dict):
            for key, value in leaves.items():
                if key not in cfg[group]:
                    cfg[group][key] = value
    return cfg


def merge_with_parent(dc: MetaseqDataclass, cfg):
    """The defaults of the component's dataclass overlaid with the values of ``cfg``; keys of ``cfg`` that the
    dataclass does not declare are kept, so configs written by other versions still load
    (metaseq/dataclass/utils.py:462-475)."""
    merged = Cfg({name: getattr(dc, name) for name in dc.field_names()})
    items = cfg.items() if isinstance(cfg, dict) else vars(cfg).items()
    for key, value in items:
        merged[key] = value
    return merged
