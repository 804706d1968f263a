"""``FusedAdam`` entry points.  The reference picks between two apex-backed classes
(metaseq/optim/fused_adam.py:11-37: V1 = ``fused_adam_cuda.adam`` per parameter with a combined scale,
V2 = ``multi_tensor_adam``); here both names resolve to the optimizer whose update is the ``msq_adamw`` kernel
(``csrc/optim.cu``): decoupled weight decay, fp32 moments (stored as scaled fp16 between steps with
``use_fp16_stats``), 16-bit parameters updated in place from an fp32
computation, and the gradient scale (1 / loss-scale x clip coefficient) folded into the kernel's read of the
gradient, so ``step(scale=...)`` needs no separate unscale pass."""
from __future__ import annotations

from typing import Optional

import torch

from .adam import Adam


class FusedAdamV1(Adam):
    """Call-compatible with the reference's V1: ``step(closure, grads, scale, grad_norms)`` where ``scale`` divides
    the gradients (combined loss scale and clipping).  Explicit ``grads`` are copied onto ``.grad`` first."""

    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, eps_inside_sqrt=False,
                 weight_decay=0.0, max_grad_norm=0.0, amsgrad=False, use_fp16_stats=False):
        if amsgrad:
            raise RuntimeError("FusedAdam does not support the AMSGrad variant.")
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, use_fp16_stats=use_fp16_stats)
        self.max_grad_norm = max_grad_norm

    def step(self, closure=None, grads=None, scale: float = 1.0, grad_norms=None, ctrl: Optional[torch.Tensor] = None):
        if grads is not None:
            flat = [p for g in self.param_groups for p in g["params"]]
            supplied = list(grads) if not isinstance(grads[0], (list, tuple)) else [x for gl in grads for x in gl]
            for p, g in zip(flat, supplied):
                if g is not None:
                    p.grad = g
        combined = float(scale)
        if self.max_grad_norm > 0 and grad_norms is not None:
            norms = grad_norms if isinstance(grad_norms, (list, tuple)) else [grad_norms]
            worst = max(float(n) for n in norms)
            clip = ((worst / combined) + 1e-6) / self.max_grad_norm
            if clip > 1:
                combined *= clip
        return super().step(closure, scale=combined, ctrl=ctrl)


FusedAdamV2 = FusedAdamV1


def get_fused_adam_class():
    """The fused optimizer class when the native kernel library can be loaded, else ``None``."""
    try:
        from metaseq_b200.ops import _lib

        return FusedAdamV1 if (_lib.kernels_available() if hasattr(_lib, "kernels_available") else True) else None
    except Exception:  # noqa: BLE001
        return None
