"""fp16 / bf16 optimizer wrappers with dynamic loss scaling.

``MemoryEfficientFP16Optimizer`` keeps parameters and gradients in 16 bits and lets the
wrapped optimizer hold fp32 moments; the factors 1/loss_scale, dp/sample_size and the clip
coefficient are folded lazily into one ``_multiply_factor`` that the fused AdamW kernel
applies to the gradient while it steps (reference: metaseq/optim/fp16_optimizer.py:322-537).
``FP16Optimizer`` keeps a flat fp32 master copy of the parameters instead (:16-320).

Step protocol (must be followed by callers, as the trainer does):
``zero_grad`` -> ``backward(loss)`` -> ``multiply_grads(c)`` -> ``clip_grad_norm(max)``
(raises ``OverflowError`` on inf/nan after adjusting the scale) -> ``step``.
"""
from __future__ import annotations

from collections import defaultdict
from itertools import chain

import torch

from metaseq_b200 import optim, utils
from metaseq_b200.dataclass.utils import get as cfg_get

from .base_optimizer import BaseOptimizer
from .dynamic_loss_scaler import DynamicLossScaler


def _build_scaler(cfg, bf16: bool):
    if bf16:
        return None
    c = cfg.common
    window = c.fp16_scale_window
    if window is None:
        uf = cfg.optimization.update_freq
        if len(uf) > 1:
            raise ValueError("--fp16-scale-window must be given explicitly when using a custom --update-freq schedule")
        dp = int(cfg.distributed_training.distributed_world_size / c.model_parallel_size)
        window = int(2 ** 14 / dp / uf[0])
    return DynamicLossScaler(init_scale=c.fp16_init_scale, scale_window=window, tolerance=c.fp16_scale_tolerance,
                             threshold=c.threshold_loss_scale, min_loss_scale=c.min_loss_scale)


def _reject_batch(grad_norm: float, max_norm: float):
    """``--skip-gradient-update-on-clip-norm``: a gradient norm above the threshold rejects the whole batch.  The
    trainer treats the exception like a loss-scale overflow: gradients are dropped and neither the update count,
    the learning-rate schedule nor the optimizer state advances (metaseq/optim/fp16_optimizer.py:186-194)."""
    raise OverflowError(f"Grad norm: {grad_norm:.2f} exceeds threshold: {max_norm:.2f}, rejecting batch.")


class _ScaledMixin:
    """Loss scaling + lazy gradient multiplier shared by both wrappers."""

    scaler = None
    _multiply_factor = 1.0

    @property
    def loss_scale(self):
        return self.scaler.loss_scale if self.scaler is not None else 1.0

    def _init_factor(self):
        self._multiply_factor = 1.0 / float(self.scaler.loss_scale) if self.scaler is not None else 1.0

    def multiply_grads(self, c):
        self._multiply_factor *= float(c) if not torch.is_tensor(c) else float(c.item())

    def _finish_norm(self, raw_norm, max_norm):
        grad_norm = self._multiply_factor * raw_norm
        if self.scaler is not None:
            gn = float(grad_norm)
            self.scaler.check_overflow(gn)
        if max_norm is not None and max_norm > 0:
            gn = float(grad_norm)
            if gn > max_norm:
                self._multiply_factor *= max_norm / (gn + 1e-6)
        return grad_norm


class MemoryEfficientFP16Optimizer(_ScaledMixin, BaseOptimizer):
    def __init__(self, cfg, params, optimizer, allow_unsupported=False, **kwargs):
        if not allow_unsupported and not optimizer.supports_memory_efficient_fp16:
            raise ValueError(f"Unsupported optimizer: {optimizer.__class__.__name__}")
        super().__init__(cfg_get(cfg, "optimizer"))
        self.wrapped_optimizer = optimizer
        self.scaler = _build_scaler(cfg, bool(cfg.common.bf16))
        self.min_loss_scale = cfg.common.min_loss_scale
        self._init_factor()

    @classmethod
    def build_optimizer(cls, cfg, params, **kwargs):
        inner = optim.build_optimizer(cfg.optimizer, params)
        return cls(cfg, params, inner, **kwargs)

    @property
    def optimizer(self):
        return self.wrapped_optimizer.optimizer

    @optimizer.setter
    def optimizer(self, optimizer):
        self.wrapped_optimizer.optimizer = optimizer

    @property
    def optimizer_config(self):
        return self.wrapped_optimizer.optimizer_config

    @property
    def lr_scheduler(self):
        return getattr(self.wrapped_optimizer, "lr_scheduler", None)

    def get_lr(self):
        return self.wrapped_optimizer.get_lr()

    def set_lr(self, lr):
        self.wrapped_optimizer.set_lr(lr)

    def all_reduce_grads(self, module):
        self.wrapped_optimizer.all_reduce_grads(module)

    def state_dict(self):
        sd = self.wrapped_optimizer.state_dict()
        if self.scaler is not None:
            sd["loss_scale"] = self.scaler.loss_scale
        return sd

    def load_state_dict(self, state_dict, optimizer_overrides=None):
        if "loss_scale" in state_dict and self.scaler is not None:
            self.scaler.loss_scale = state_dict["loss_scale"]
        sd = {k: v for k, v in state_dict.items() if k != "loss_scale"}
        self.wrapped_optimizer.load_state_dict(sd, optimizer_overrides)
        # torch.optim casts loaded state to the dtype of its parameter.  Here the parameters are 16-bit and the
        # moments fp32: a second moment of 1e-9 does not survive fp16, and the first update after a resume would
        # divide by eps alone.  Put the saved tensors back in their saved dtype (they move to the device at the
        # next step).
        saved_groups = sd.get("param_groups", [])
        saved_ids = [i for g in saved_groups for i in g["params"]]
        params = [p for g in self.optimizer.param_groups for p in g["params"]]
        by_id = dict(zip(saved_ids, params))
        for key, st in sd.get("state", {}).items():
            param = by_id.get(key)
            if param is None:
                continue
            self.optimizer.state[param] = {
                k: (v.detach().clone() if torch.is_tensor(v) and v.is_floating_point() else v) for k, v in st.items()}

    def backward(self, loss):
        if self.scaler is not None:
            loss = self.scaler.scale(loss)
        loss.backward()

    def _unscale_grads(self):
        if self._multiply_factor != 1.0:
            self.wrapped_optimizer.multiply_grads(self._multiply_factor)
            self._multiply_factor = 1.0

    def clip_grad_norm(self, max_norm, norm_type="l2", aggregate_norm_fn=None, skip_gradient_update_on_clip_norm=False):
        raw = self.wrapped_optimizer.clip_grad_norm(0, norm_type, aggregate_norm_fn)
        grad_norm = self._multiply_factor * raw
        if self.scaler is not None:
            gn = float(grad_norm)  # the one device-to-host read of the step
            self.scaler.check_overflow(gn)
        else:
            gn = None
        if max_norm is not None and max_norm > 0:
            gn = float(grad_norm) if gn is None else gn
            if skip_gradient_update_on_clip_norm and self.scaler is not None and gn > max_norm:
                _reject_batch(gn, max_norm)
            self._multiply_factor *= min(1.0, max_norm / (gn + 1e-6))
        return grad_norm

    def step(self, closure=None, groups=None):
        if getattr(self, "supports_step_with_scale", False):
            self.wrapped_optimizer.step(closure, scale=1.0 / self._multiply_factor)
        else:
            self._unscale_grads()
            self.wrapped_optimizer.step(closure)
        if self.scaler is not None:
            self.scaler.update()

    def zero_grad(self):
        self.wrapped_optimizer.zero_grad()
        self._init_factor()

    @property
    def supports_flat_params(self):
        return self.wrapped_optimizer.supports_flat_params

    @property
    def supports_step_with_scale(self):
        return self.wrapped_optimizer.supports_step_with_scale


class FP16Optimizer(_ScaledMixin, BaseOptimizer):
    """16-bit model parameters with an fp32 master copy (one flat tensor per device) that the
    wrapped optimizer updates; gradients are copied fp16 -> fp32 before the step and parameters
    fp32 -> fp16 after it."""

    def __init__(self, cfg, params, fp32_optimizer, fp32_params, **kwargs):
        super().__init__(cfg_get(cfg, "optimizer"))
        self.fp16_params = params
        self.fp32_optimizer = fp32_optimizer
        self.fp32_params = fp32_params
        self.scaler = _build_scaler(cfg, bool(cfg.common.bf16))
        self.min_loss_scale = cfg.common.min_loss_scale
        self._needs_sync = True
        self._init_factor()

    @classmethod
    def build_fp32_params(cls, params, flatten=True):
        if flatten:
            devices = defaultdict(list)
            for p in params:
                devices[p.device].append(p)
            out = {}
            for dev, plist in devices.items():
                total = sum(p.data.numel() for p in plist)
                flat = plist[0].new_zeros(total, dtype=torch.float32)
                off = 0
                for p in plist:
                    n = p.data.numel()
                    flat[off:off + n].copy_(p.data.view(-1))
                    off += n
                flat = torch.nn.Parameter(flat)
                flat.grad = flat.data.new_zeros(total)
                out[dev] = flat
            return out
        out = []
        for p in params:
            p32 = torch.nn.Parameter(p.data.float())
            p32.grad = torch.zeros_like(p32.data)
            if hasattr(p, "param_group"):
                p32.param_group = p.param_group
            out.append(p32)
        return out

    @classmethod
    def build_optimizer(cls, cfg, params, **kwargs):
        flatten = not getattr(cfg.common, "fp16_no_flatten_grads", False)
        fp32_params = cls.build_fp32_params(params, flatten=flatten)
        inner = optim.build_optimizer(cfg.optimizer, list(fp32_params.values()) if flatten else fp32_params)
        if flatten and not inner.supports_flat_params:
            raise RuntimeError(f"chosen optimizer {inner.__class__.__name__} does not support flat params, "
                               "please set --fp16-no-flatten-grads")
        return cls(cfg, params, inner, fp32_params, **kwargs)

    @property
    def has_flat_params(self):
        return isinstance(self.fp32_params, dict)

    @property
    def optimizer(self):
        return self.fp32_optimizer.optimizer

    @optimizer.setter
    def optimizer(self, optimizer):
        self.fp32_optimizer.optimizer = optimizer

    @property
    def optimizer_config(self):
        return self.fp32_optimizer.optimizer_config

    @property
    def lr_scheduler(self):
        return getattr(self.fp32_optimizer, "lr_scheduler", None)

    def get_lr(self):
        return self.fp32_optimizer.get_lr()

    def set_lr(self, lr):
        self.fp32_optimizer.set_lr(lr)

    def all_reduce_grads(self, module):
        self.fp32_optimizer.all_reduce_grads(module)

    def state_dict(self):
        sd = self.fp32_optimizer.state_dict()
        if self.scaler is not None:
            sd["loss_scale"] = self.scaler.loss_scale
        return sd

    def load_state_dict(self, state_dict, optimizer_overrides=None):
        if "loss_scale" in state_dict and self.scaler is not None:
            self.scaler.loss_scale = state_dict["loss_scale"]
        sd = {k: v for k, v in state_dict.items() if k != "loss_scale"}
        self.fp32_optimizer.load_state_dict(sd, optimizer_overrides)

    def backward(self, loss):
        if self.scaler is not None:
            loss = self.scaler.scale(loss)
        loss.backward()
        self._needs_sync = True

    def _sync_fp16_grads_to_fp32(self):
        if not self._needs_sync:
            return
        if self.has_flat_params:
            devices = defaultdict(list)
            for p in self.fp16_params:
                if p.requires_grad:
                    devices[p.device].append(p)
            for dev, plist in devices.items():
                flat = self.fp32_params[dev]
                off = 0
                for p in plist:
                    n = p.data.numel()
                    if p.grad is not None:
                        flat.grad.data[off:off + n].copy_(p.grad.data.view(-1))
                    else:
                        flat.grad.data[off:off + n].zero_()
                    off += n
        else:
            for p, p32 in zip(self.fp16_params, self.fp32_params):
                if not p.requires_grad:
                    continue
                if p.grad is not None:
                    if p32.grad is None:
                        p32.grad = p.grad.data.float()
                    else:
                        p32.grad.data.copy_(p.grad.data)
                else:
                    p32.grad = torch.zeros_like(p.data, dtype=torch.float)
        self._needs_sync = False

    def _sync_fp32_params_to_fp16(self):
        if self.has_flat_params:
            devices = defaultdict(list)
            for p in self.fp16_params:
                devices[p.device].append(p)
            for dev, plist in devices.items():
                flat = self.fp32_params[dev]
                off = 0
                for p in plist:
                    n = p.data.numel()
                    p.data.copy_(flat.data[off:off + n].view_as(p.data))
                    off += n
        else:
            for p, p32 in zip(self.fp16_params, self.fp32_params):
                if p.requires_grad:
                    p.data.copy_(p32.data)

    def _unscale_grads(self):
        self._sync_fp16_grads_to_fp32()
        if self._multiply_factor != 1.0:
            self.fp32_optimizer.multiply_grads(self._multiply_factor)
            self._multiply_factor = 1.0

    def clip_grad_norm(self, max_norm, norm_type="l2", aggregate_norm_fn=None, skip_gradient_update_on_clip_norm=False):
        self._sync_fp16_grads_to_fp32()
        raw = self.fp32_optimizer.clip_grad_norm(0, norm_type, aggregate_norm_fn)
        grad_norm = self._multiply_factor * raw
        if self.scaler is not None:
            self.scaler.check_overflow(float(grad_norm))
        if max_norm is not None and max_norm > 0:
            gn = float(grad_norm)
            if skip_gradient_update_on_clip_norm and self.scaler is not None and gn > max_norm:
                _reject_batch(gn, max_norm)
            self._multiply_factor *= min(1.0, max_norm / (gn + 1e-6))
        return grad_norm

    def step(self, closure=None, groups=None):
        self._sync_fp16_grads_to_fp32()
        if getattr(self.fp32_optimizer, "supports_step_with_scale", False):
            self.fp32_optimizer.step(closure, scale=(1.0 / self._multiply_factor))
        else:
            self._unscale_grads()
            self.fp32_optimizer.step(closure)
        if self.scaler is not None:
            self.scaler.update()
        self._sync_fp32_params_to_fp16()

    def zero_grad(self):
        for p in self.fp16_params:
            p.grad = None
        if self.has_flat_params:
            for flat in self.fp32_params.values():
                flat.grad.zero_()
        else:
            for p32 in self.fp32_params:
                if p32.grad is not None:
                    p32.grad.zero_()
        self._needs_sync = False
        self._init_factor()

    @property
    def supports_flat_params(self):
        return self.fp32_optimizer.supports_flat_params
