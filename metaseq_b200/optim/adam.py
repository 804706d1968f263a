"""AdamW (decoupled weight decay).  State is always fp32; 16-bit parameters are updated
through an fp32 view of themselves (no persistent master copy), which is what lets the
memory-efficient fp16 wrapper work.  On CUDA every parameter tensor is stepped by one fused
kernel that also applies the 1/scale factor to the gradient; on CPU the same math runs as
PyTorch ops.  Reference: metaseq/optim/adam.py:42-218 and the apex kernel it prefers
(metaseq/modules/apex/fused_adam_cuda_kernel.cu:66-102)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, List, Optional

import torch
import torch.optim

from metaseq_b200.dataclass.configs import MetaseqDataclass, opt
from metaseq_b200.ops import functional as ops

from . import register_optimizer
from .base_optimizer import BaseOptimizer


@dataclass
class MetaseqAdamConfig(MetaseqDataclass):
    lr: Any = opt(factory=lambda: [0.25], help="learning rate (mirrors --lr)", link="optimization.lr")
    adam_betas: Any = opt("(0.9, 0.999)", "betas for Adam optimizer")
    adam_eps: float = opt(1e-8, "epsilon for Adam optimizer")
    weight_decay: float = opt(0.0, "weight decay")
    use_old_adam: Optional[bool] = opt(False, "use the PyTorch-ops implementation even on a GPU")
    fp16_adam_stats: bool = opt(False, "kept for command-line compatibility; moments are stored in fp32")
    block_wise: bool = opt(False, "kept for command-line compatibility")


@register_optimizer("adam", dataclass=MetaseqAdamConfig)
class MetaseqAdam(BaseOptimizer):
    def __init__(self, cfg, params):
        super().__init__(cfg)
        self._optimizer = Adam(params, **self.optimizer_config)

    @property
    def optimizer_config(self):
        betas = self.cfg.adam_betas
        if isinstance(betas, str):
            betas = eval(betas)
        lr = self.cfg.lr[0] if isinstance(getattr(self.cfg, "lr", None), (list, tuple)) else getattr(self.cfg, "lr", 1e-3)
        return {
            "lr": lr,
            "betas": tuple(betas),
            "eps": self.cfg.adam_eps,
            "weight_decay": self.cfg.weight_decay,
            "use_kernels": not getattr(self.cfg, "use_old_adam", False),
        }


class Adam(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, use_kernels=True):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.use_kernels = use_kernels

    @property
    def supports_memory_efficient_fp16(self):
        return True

    @property
    def supports_flat_params(self):
        return True

    @property
    def supports_step_with_scale(self):
        return True

    @torch.no_grad()
    def step(self, closure=None, scale: float = 1.0, ctrl: Optional[torch.Tensor] = None):
        """``scale``: gradients are divided by it inside the update.  ``ctrl``: optional device
        control block (grad multiplier + skip flag) that replaces ``scale``."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            batched = {}  # (step, param dtype, grad dtype, device) -> [(p, g, m, v)]: one launch each
            for p in group["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                if grad.is_sparse:
                    raise RuntimeError("Adam does not support sparse gradients")
                state = self.state[p]
                if len(state) == 0:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                else:
                    state["exp_avg"] = state["exp_avg"].to(device=p.device, dtype=torch.float32)
                    state["exp_avg_sq"] = state["exp_avg_sq"].to(device=p.device, dtype=torch.float32)
                state["step"] += 1
                m, v = state["exp_avg"], state["exp_avg_sq"]
                if p.is_cuda and self.use_kernels and p.is_contiguous() and grad.is_contiguous() \
                        and ops.get_backend() != "torch":
                    batched.setdefault((state["step"], p.dtype, grad.dtype, p.device), []).append((p.data, grad, m, v))
                    continue
                g32 = grad.float()
                if ctrl is not None:
                    if float(ctrl[1]) != 0:
                        state["step"] -= 1
                        continue
                    g32 = g32 * float(ctrl[0])
                elif scale != 1.0:
                    g32 = g32 / scale
                p32 = p.data.float() if p.dtype != torch.float32 else p.data
                m.mul_(beta1).add_(g32, alpha=1 - beta1)
                v.mul_(beta2).addcmul_(g32, g32, value=1 - beta2)
                denom = v.sqrt().add_(group["eps"])
                bc1 = 1 - beta1 ** state["step"]
                bc2 = 1 - beta2 ** state["step"]
                step_size = group["lr"] * math.sqrt(bc2) / bc1
                if group["weight_decay"] != 0:
                    p32.add_(p32, alpha=-group["weight_decay"] * group["lr"])
                p32.addcdiv_(m, denom, value=-step_size)
                if p.dtype != torch.float32:
                    p.data.copy_(p32)
            for (step, _, _, device), items in batched.items():
                local_ctrl = ctrl
                if local_ctrl is None and scale != 1.0:
                    local_ctrl = self._scale_ctrl(device, scale)
                kw = dict(lr=group["lr"], beta1=beta1, beta2=beta2, eps=group["eps"],
                          weight_decay=group["weight_decay"], step=step, ctrl=local_ctrl)
                if len(items) == 1:
                    ops.adamw_step(*items[0], **kw)
                else:
                    ops.adamw_step_multi(items, **kw)
        return loss

    _ctrl_cache = {}

    def _scale_ctrl(self, device, scale):
        key = (str(device), float(scale))
        c = Adam._ctrl_cache.get(key)
        if c is None:
            if len(Adam._ctrl_cache) > 64:
                Adam._ctrl_cache.clear()
            c = torch.tensor([1.0 / scale, 0.0, 0.0, 1.0], dtype=torch.float32, device=device)
            Adam._ctrl_cache[key] = c
        return c
