"""Thin wrapper protocol around a ``torch.optim.Optimizer`` (reference:
metaseq/optim/base_optimizer.py:12-181)."""
from __future__ import annotations

import torch

from metaseq_b200 import utils
from metaseq_b200.dataclass.utils import gen_parser_from_dataclass


def _capability(name: str, doc: str):
    """A read-only flag that mirrors the same-named attribute of the wrapped torch optimizer (False if absent)."""
    return property(lambda self: getattr(self.optimizer, name, False), doc=doc)


class BaseOptimizer:
    """What the trainer and the half-precision wrappers expect of an optimizer: the wrapped ``torch.optim``
    object as ``optimizer``, learning-rate access, gradient scaling / clipping, ``step(scale=...)`` and a few
    capability flags."""

    def __init__(self, cfg):
        self.cfg = cfg

    # -- construction ------------------------------------------------------------------------------
    @classmethod
    def add_args(cls, parser):
        declared = getattr(cls, "__dataclass", None)
        if declared is not None:
            gen_parser_from_dataclass(parser, declared())

    @classmethod
    def build_optimizer(cls, cfg, params, *a, **kw):
        return cls(cfg, params, *a, **kw)

    # -- the wrapped optimizer ---------------------------------------------------------------------
    @property
    def optimizer(self):
        try:
            return self._optimizer
        except AttributeError:
            raise NotImplementedError from None

    @optimizer.setter
    def optimizer(self, value):
        self._optimizer = value

    @property
    def optimizer_config(self):
        """Keyword arguments from which an equivalent optimizer can be rebuilt (checkpoints store them)."""
        raise NotImplementedError

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def params(self):
        return (p for group in self.param_groups for p in group["params"])

    def __getstate__(self):
        return self._optimizer.__getstate__()

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, state_dict, optimizer_overrides=None):
        """Restores the saved state, then lets ``optimizer_overrides`` replace group settings (a new learning
        rate for a resumed run, for instance)."""
        self.optimizer.load_state_dict(state_dict)
        for group in self.param_groups if optimizer_overrides else ():
            group.update(optimizer_overrides)

    def broadcast_global_state_dict(self, state_dict):
        spread = getattr(self.optimizer, "broadcast_global_state_dict", None)
        return spread(state_dict) if spread is not None else state_dict

    # -- learning rate -----------------------------------------------------------------------------
    def get_lr(self):
        return self.param_groups[0]["lr"]

    def set_lr(self, lr):
        for group in self.param_groups:
            group["lr"] = lr

    # -- gradients ---------------------------------------------------------------------------------
    def backward(self, loss):
        loss.backward()

    def all_reduce_grads(self, module):
        reduce = getattr(module, "all_reduce_grads", None)
        if reduce is not None:
            reduce()

    def multiply_grads(self, c):
        for p in self.params:
            if p.grad is not None:
                p.grad.data.mul_(c.to(p.grad.device) if torch.is_tensor(c) else c)

    def clip_grad_norm(self, max_norm, norm_type="l2", aggregate_norm_fn=None, **kwargs):
        return utils.clip_grad_norm_(self.params, max_norm, norm_type, aggregate_norm_fn)

    def zero_grad(self):
        for p in self.params:
            p.grad = None
        self.optimizer.zero_grad()

    # -- update ------------------------------------------------------------------------------------
    def step(self, closure=None, scale=1.0, groups=None):
        """One update from gradients that are ``scale`` times too large: optimizers that take the factor divide
        inside their kernel, for the others the gradients are rescaled first."""
        if self.supports_step_with_scale:
            return self.optimizer.step(closure, scale=scale)
        if scale != 1.0:
            self.multiply_grads(1.0 / scale)
        return self.optimizer.step(closure)

    def average_params(self):
        pass

    supports_memory_efficient_fp16 = _capability(
        "supports_memory_efficient_fp16", "Updates 16-bit parameters in fp32 arithmetic without an fp32 copy.")
    supports_step_with_scale = _capability("supports_step_with_scale", "``step`` takes the gradient scale.")
    supports_flat_params = _capability("supports_flat_params", "Works on one flat buffer per dtype.")
    supports_groups = _capability("supports_groups", "Honours parameter groups with their own hyper-parameters.")


class LegacyOptimizer(BaseOptimizer):
    """Base for optimizers configured by an argparse namespace instead of a dataclass
    (metaseq/optim/base_optimizer.py:179-181)."""

    def __init__(self, args):
        super().__init__(args)
        self.args = args
