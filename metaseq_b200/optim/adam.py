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
    fp16_adam_stats: bool = opt(False, "store the moments in fp16 with a per-tensor scale (halves optimizer state)")
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
            "use_fp16_stats": bool(getattr(self.cfg, "fp16_adam_stats", False)),
        }


class Adam(torch.optim.Optimizer):
    """AdamW with fp32 arithmetic.  With ``use_fp16_stats`` the two moments are kept between steps as fp16 tensors
    with one fp32 scale each (``exp_avg_scale``, ``exp_avg_sq_scale``: the tensor's largest magnitude mapped to the
    top of the fp16 range), expanded to fp32 for the update and compressed again after it: the scheme of the
    reference's fused optimizer (metaseq/optim/fused_adam.py:189-249)."""

    FLOAT16_MAX = 65504.0

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, use_kernels=True,
                 use_fp16_stats=False, amsgrad=False):
        if amsgrad:
            raise NotImplementedError("the AMSGrad variant (running maximum of the second moment) is not built; "
                                      "the OPT recipes do not use it")
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.use_kernels = use_kernels
        self.use_fp16_stats = use_fp16_stats

    def _expand_stats(self, state, p):
        """fp32 working copies of the two moments of ``p``."""
        if not self.use_fp16_stats:
            state["exp_avg"] = state["exp_avg"].to(device=p.device, dtype=torch.float32)
            state["exp_avg_sq"] = state["exp_avg_sq"].to(device=p.device, dtype=torch.float32)
            return state["exp_avg"], state["exp_avg_sq"]
        out = []
        for name in ("exp_avg", "exp_avg_sq"):
            t = state[name].to(device=p.device)
            sc = state.get(name + "_scale")
            if sc is not None:  # a loader may have cast the stored fp16 values to another dtype: the values stand
                sc = sc.to(device=p.device, dtype=torch.float32) if torch.is_tensor(sc) else float(sc)
                t = t.float() * sc
            else:  # state written without compression (a checkpoint of an fp32-moment run, or a resharded one)
                t = t.float()
            out.append(t)
        return out[0], out[1]

    def _compress_stats(self, state, m, v):
        for name, t in (("exp_avg", m), ("exp_avg_sq", v)):
            # the reference adds 1e-8 here, which swamps the second moments of small gradients (1e-12 and below)
            # into fp16 subnormals; the floor only has to keep an all-zero tensor from dividing by zero
            sc = (t.abs().max().float() / self.FLOAT16_MAX).clamp_min(1e-30)
            state[name + "_scale"] = sc
            state[name] = (t / sc).half()

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
            compress = []  # (state, m, v) whose fp32 working copies go back to fp16 after the update
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
                state["step"] += 1
                m, v = self._expand_stats(state, p)
                if self.use_fp16_stats:
                    compress.append((state, m, v))
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
            for state, m, v in compress:
                self._compress_stats(state, m, v)
        return loss

    def _scale_ctrl(self, device, scale):
        """Device control block [gradient multiplier, skip flag, norm, clip coefficient] for a host-side ``scale``:
        one pinned staging buffer and one device buffer per optimizer and device, refilled with an asynchronous copy
        (the scale changes with every clipped update, so nothing is cached by value)."""
        bufs = self.__dict__.setdefault("_ctrl_bufs", {})
        entry = bufs.get(str(device))
        if entry is None:
            host = torch.zeros(4, dtype=torch.float32)
            if torch.cuda.is_available():
                host = host.pin_memory()
            entry = (host, torch.zeros(4, dtype=torch.float32, device=device), [None])
            bufs[str(device)] = entry
        host, dev, pending = entry
        if pending[0] is not None:
            pending[0].synchronize()  # the previous copy out of the staging buffer has to be done before a refill
        host[0], host[1], host[2], host[3] = 1.0 / scale, 0.0, 0.0, 1.0
        dev.copy_(host, non_blocking=True)
        if dev.is_cuda:
            pending[0] = torch.cuda.Event()
            pending[0].record()
        return dev
