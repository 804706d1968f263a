"""Task registry (``--task``); reference: metaseq/tasks/__init__.py:24-101."""
from __future__ import annotations

import argparse

from .base_task import BaseTask, LegacyTask

TASK_DATACLASS_REGISTRY = {}
TASK_REGISTRY = {}
TASK_CLASS_NAMES = set()


def setup_task(cfg, **kwargs):
    """``cfg`` is the task node of the config (a ``Cfg`` with ``_name``, or a flat namespace
    with ``task``)."""
    name = cfg.get("_name") if hasattr(cfg, "get") else getattr(cfg, "_name", None)
    if name is None:
        name = getattr(cfg, "task", None)
    task = TASK_REGISTRY.get(name)
    assert task is not None, f"Could not infer task type from {cfg}. Available tasks: {sorted(TASK_REGISTRY)}"
    return task.setup_task(cfg, **kwargs)


def register_task(name, dataclass=None):
    def wrap(cls):
        if name in TASK_REGISTRY:
            raise ValueError(f"Cannot register duplicate task ({name})")
        if not issubclass(cls, BaseTask):
            raise ValueError(f"Task ({name}: {cls.__name__}) must extend BaseTask")
        if cls.__name__ in TASK_CLASS_NAMES:
            raise ValueError(f"Cannot register task with duplicate class name ({cls.__name__})")
        TASK_REGISTRY[name] = cls
        TASK_CLASS_NAMES.add(cls.__name__)
        if dataclass is not None:
            cls.__dataclass = dataclass
            TASK_DATACLASS_REGISTRY[name] = dataclass
            from metaseq_b200.dataclass.initialize import ConfigStore

            ConfigStore.instance().store(name=name, group="task", node=dataclass)
        return cls

    return wrap


def get_task(name):
    return TASK_REGISTRY[name]


from . import dummy_lm, language_modeling, streaming_language_modeling, streaming_finetune_language_modeling  # noqa: E402,F401
