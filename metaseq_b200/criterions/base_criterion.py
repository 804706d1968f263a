"""Base class of loss functions (reference: metaseq/criterions/base_criterion.py).

A criterion is built from its config by matching the constructor's parameter names: ``task`` and ``cfg`` are passed
as such, any other name is looked up in the config, and a parameter that is not there must have a default.
``forward(model, sample)`` returns ``(loss, sample_size, logging_output)``; ``reduce_metrics`` turns the logging
outputs of all ranks into logged scalars.
"""
from __future__ import annotations

import inspect
from typing import Any, Dict, List

from torch.nn.modules.loss import _Loss

from metaseq_b200.dataclass.utils import gen_parser_from_dataclass

_UNSUPPORTED = (inspect.Parameter.POSITIONAL_ONLY, inspect.Parameter.VAR_POSITIONAL, inspect.Parameter.VAR_KEYWORD)


def _lookup(cfg, name: str):
    """``(found, value)`` of ``name`` in a config that is a mapping or an object with attributes."""
    if isinstance(cfg, dict):
        return (name in cfg), cfg.get(name)
    return hasattr(cfg, name), getattr(cfg, name, None)


class BaseCriterion(_Loss):
    def __init__(self, task):
        super().__init__()
        self.task = task
        dictionary = getattr(task, "target_dictionary", None)
        if hasattr(task, "target_dictionary"):
            self.padding_idx = dictionary.pad() if dictionary is not None else -100

    @classmethod
    def add_args(cls, parser):
        """Adds the flags of the dataclass this criterion was registered with."""
        declared = getattr(cls, "__dataclass", None)
        if declared is not None:
            gen_parser_from_dataclass(parser, declared())

    @classmethod
    def build_criterion(cls, cfg, task):
        given = {"task": task, "cfg": cfg}
        kwargs = {}
        for param in inspect.signature(cls).parameters.values():
            if param.kind in _UNSUPPORTED:
                raise NotImplementedError(f"{param.kind} not supported")
            if param.name in given:
                kwargs[param.name] = given[param.name]
                continue
            found, value = _lookup(cfg, param.name)
            if found:
                kwargs[param.name] = value
            elif param.default is param.empty:
                raise NotImplementedError(f"Unable to infer Criterion argument {param.name}")
        return cls(**kwargs)

    def forward(self, model, sample, reduce=True):
        raise NotImplementedError

    @staticmethod
    def reduce_metrics(logging_outputs: List[Dict[str, Any]]) -> None:
        raise NotImplementedError

    @staticmethod
    def logging_outputs_can_be_summed() -> bool:
        """True lets the trainer sum the logging outputs with one all-reduce instead of gathering them."""
        return False
