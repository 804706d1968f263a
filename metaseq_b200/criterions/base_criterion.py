"""Criterion base class (reference: metaseq/criterions/base_criterion.py)."""
from __future__ import annotations

import inspect
from typing import Any, Dict, List

from torch.nn.modules.loss import _Loss

from metaseq_b200.dataclass.utils import gen_parser_from_dataclass


class BaseCriterion(_Loss):
    def __init__(self, task):
        super().__init__()
        self.task = task
        if hasattr(task, "target_dictionary"):
            tgt = task.target_dictionary
            self.padding_idx = tgt.pad() if tgt is not None else -100

    @classmethod
    def add_args(cls, parser):
        dc = getattr(cls, "__dataclass", None)
        if dc is not None:
            gen_parser_from_dataclass(parser, dc())

    @classmethod
    def build_criterion(cls, cfg, task):
        init_args = {}
        for p in inspect.signature(cls).parameters.values():
            if p.kind in (p.POSITIONAL_ONLY, p.VAR_POSITIONAL, p.VAR_KEYWORD):
                raise NotImplementedError(f"{p.kind} not supported")
            if p.name == "task":
                init_args["task"] = task
            elif p.name == "cfg":
                init_args["cfg"] = cfg
            elif hasattr(cfg, p.name) or (isinstance(cfg, dict) and p.name in cfg):
                init_args[p.name] = cfg[p.name] if isinstance(cfg, dict) else getattr(cfg, p.name)
            elif p.default != p.empty:
                pass
            else:
                raise NotImplementedError(f"Unable to infer Criterion argument {p.name}")
        return cls(**init_args)

    def forward(self, model, sample, reduce=True):
        """Returns ``(loss, sample_size, logging_output)``."""
        raise NotImplementedError

    @staticmethod
    def reduce_metrics(logging_outputs: List[Dict[str, Any]]) -> None:
        raise NotImplementedError

    @staticmethod
    def logging_outputs_can_be_summed() -> bool:
        return False
