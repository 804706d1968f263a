"""SGD with decoupled weight decay (``--optimizer sgdw``) and plain SGD (reference:
metaseq/optim/sgd.py)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.optim

from metaseq_b200.dataclass.configs import MetaseqDataclass, opt

from . import register_optimizer
from .base_optimizer import BaseOptimizer


@dataclass
class SGDConfig(MetaseqDataclass):
    lr: Any = opt(factory=lambda: [0.25], help="learning rate (mirrors --lr)", link="optimization.lr")
    momentum: float = opt(0.0, "momentum factor")
    weight_decay: float = opt(0.0, "weight decay")


class SGDW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0, weight_decay=0.0, nesterov=False):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov))

    @property
    def supports_memory_efficient_fp16(self):
        return True

    @property
    def supports_flat_params(self):
        return True

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                p32 = p.data.float() if p.dtype != torch.float32 else p.data
                if group["weight_decay"] != 0:
                    p32.mul_(1 - group["lr"] * group["weight_decay"])
                if group["momentum"] != 0:
                    st = self.state[p]
                    buf = st.get("momentum_buffer")
                    if buf is None:
                        buf = st["momentum_buffer"] = g.clone()
                    else:
                        buf.mul_(group["momentum"]).add_(g, alpha=1 - group.get("dampening", 0))
                    g = g.add(buf, alpha=group["momentum"]) if group.get("nesterov", False) else buf
                p32.add_(g, alpha=-group["lr"])
                if p.dtype != torch.float32:
                    p.data.copy_(p32)
        return loss


@register_optimizer("sgdw", dataclass=SGDConfig)
class MetaseqSGDW(BaseOptimizer):
    def __init__(self, cfg, params):
        super().__init__(cfg)
        self._optimizer = SGDW(params, **self.optimizer_config)

    @property
    def optimizer_config(self):
        lr = self.cfg.lr[0] if isinstance(getattr(self.cfg, "lr", None), (list, tuple)) else getattr(self.cfg, "lr", 1e-3)
        return {"lr": lr, "momentum": self.cfg.momentum, "weight_decay": self.cfg.weight_decay}


@register_optimizer("sgd", dataclass=SGDConfig)
class MetaseqSGD(BaseOptimizer):
    def __init__(self, cfg, params):
        super().__init__(cfg)
        self._optimizer = torch.optim.SGD(params, **self.optimizer_config)

    @property
    def optimizer_config(self):
        lr = self.cfg.lr[0] if isinstance(getattr(self.cfg, "lr", None), (list, tuple)) else getattr(self.cfg, "lr", 1e-3)
        return {"lr": lr, "momentum": self.cfg.momentum, "weight_decay": self.cfg.weight_decay}
