"""Thin wrapper protocol around a ``torch.optim.Optimizer`` (reference:
metaseq/optim/base_optimizer.py:12-181)."""
from __future__ import annotations

import torch

from metaseq_b200 import utils
from metaseq_b200.dataclass.utils import gen_parser_from_dataclass


class BaseOptimizer:
    def __init__(self, cfg):
        self.cfg = cfg

    @classmethod
    def add_args(cls, parser):
        dc = getattr(cls, "__dataclass", None)
        if dc is not None:
            gen_parser_from_dataclass(parser, dc())

    @classmethod
    def build_optimizer(cls, cfg, params, *a, **kw):
        return cls(cfg, params, *a, **kw)

    @property
    def optimizer(self):
        if not hasattr(self, "_optimizer"):
            raise NotImplementedError
        return self._optimizer

    @optimizer.setter
    def optimizer(self, optimizer):
        self._optimizer = optimizer

    @property
    def optimizer_config(self):
        raise NotImplementedError

    @property
    def params(self):
        for group in self.param_groups:
            for p in group["params"]:
                yield p

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def __getstate__(self):
        return self._optimizer.__getstate__()

    def get_lr(self):
        return self.param_groups[0]["lr"]

    def set_lr(self, lr):
        for g in self.param_groups:
            g["lr"] = lr

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, state_dict, optimizer_overrides=None):
        """Loads state; the current optimizer configuration (lr etc.) overrides what was
        saved, then ``optimizer_overrides`` is applied on top."""
        self.optimizer.load_state_dict(state_dict)
        if optimizer_overrides:
            for g in self.param_groups:
                g.update(optimizer_overrides)

    def backward(self, loss):
        loss.backward()

    def all_reduce_grads(self, module):
        if hasattr(module, "all_reduce_grads"):
            module.all_reduce_grads()

    def multiply_grads(self, c):
        for p in self.params:
            if p.grad is not None:
                if torch.is_tensor(c):
                    c = c.to(p.grad.device)
                p.grad.data.mul_(c)

    def clip_grad_norm(self, max_norm, norm_type="l2", aggregate_norm_fn=None, **kwargs):
        return utils.clip_grad_norm_(self.params, max_norm, norm_type, aggregate_norm_fn)

    def step(self, closure=None, scale=1.0, groups=None):
        if self.supports_step_with_scale:
            self.optimizer.step(closure, scale=scale)
        else:
            if scale != 1.0:
                self.multiply_grads(1.0 / scale)
            self.optimizer.step(closure)

    def zero_grad(self):
        for p in self.params:
            p.grad = None
        self.optimizer.zero_grad()

    @property
    def supports_memory_efficient_fp16(self):
        return getattr(self.optimizer, "supports_memory_efficient_fp16", False)

    @property
    def supports_step_with_scale(self):
        return getattr(self.optimizer, "supports_step_with_scale", False)

    @property
    def supports_flat_params(self):
        return getattr(self.optimizer, "supports_flat_params", False)

    @property
    def supports_groups(self):
        """Whether parameter groups with their own hyper-parameters are honoured."""
        return getattr(self.optimizer, "supports_groups", False)

    def average_params(self):
        pass

    def broadcast_global_state_dict(self, state_dict):
        if hasattr(self.optimizer, "broadcast_global_state_dict"):
            return self.optimizer.broadcast_global_state_dict(state_dict)
        return state_dict



class LegacyOptimizer(BaseOptimizer):
    """Base for optimizers configured by an argparse namespace instead of a dataclass
    (metaseq/optim/base_optimizer.py:179-181)."""

    def __init__(self, args):
        super().__init__(args)
        self.args = args
