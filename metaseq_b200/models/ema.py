"""Exponential moving average of the model parameters (reference: metaseq/models/ema/ema.py:32-204).
The shadow copy can be kept in fp32 while the model trains in 16 bits; updates start after
``ema_start_update`` and run every ``ema_update_freq`` updates."""
from __future__ import annotations

import copy
import logging

import torch

logger = logging.getLogger(__name__)


class EMA:
    def __init__(self, model, config, device=None, skip_keys=None):
        self.decay = config.ema_decay
        self.model = copy.deepcopy(model)
        self.model.requires_grad_(False)
        self.config = config
        self.skip_keys = skip_keys or set()
        self.fp32_params = {}
        if device is not None:
            logger.info(f"Copying EMA model to device {device}")
            self.model = self.model.to(device=device)
        if self.config.ema_fp32:
            self.build_fp32_params()
        self.update_freq_counter = 0

    def get_model(self):
        return self.model

    def build_fp32_params(self, state_dict=None):
        if not self.config.ema_fp32:
            raise RuntimeError("build_fp32_params should not be called if ema_fp32=False.")
        if state_dict is None:
            state_dict = self.model.state_dict()

        def _to_float(t):
            return t.float() if torch.is_floating_point(t) else t

        for k, v in state_dict.items():
            if k in self.fp32_params:
                self.fp32_params[k].copy_(v)
            else:
                self.fp32_params[k] = _to_float(v).clone()

    def restore(self, state_dict, build_fp32_params=False):
        self.model.load_state_dict(state_dict, strict=False)
        if build_fp32_params:
            self.build_fp32_params(state_dict)

    def _set_decay(self, decay):
        self.decay = decay

    def get_decay(self):
        return self.decay

    def _step_internal(self, new_model, updates=None):
        decay = self.decay
        ema_state = self.fp32_params if self.config.ema_fp32 else self.model.state_dict()
        out = {}
        for key, param in new_model.state_dict().items():
            if isinstance(param, dict):
                continue
            if key not in ema_state:
                ema_state[key] = param.float().clone() if param.ndim >= 1 else copy.deepcopy(param)
            ema_param = ema_state[key]
            if key in self.skip_keys or not torch.is_floating_point(param):
                ema_param = param.to(dtype=ema_param.dtype).clone() if torch.is_tensor(ema_param) else param
            else:
                ema_param.mul_(decay)
                ema_param.add_(param.to(dtype=ema_param.dtype, device=ema_param.device), alpha=1 - decay)
            out[key] = ema_param
        self.restore(out, build_fp32_params=False)

    def step(self, new_model, updates=None):
        """Called once per optimizer update."""
        self._set_decay(0 if updates is not None and updates < self.config.ema_start_update else self.config.ema_decay)
        if updates is not None and self.config.ema_update_freq > 1:
            self.update_freq_counter += 1
            if self.update_freq_counter >= self.config.ema_update_freq:
                self._step_internal(new_model, updates)
                self.update_freq_counter = 0
        else:
            self._step_internal(new_model, updates)

    def reverse(self, model):
        """Loads the averaged parameters into ``model`` (for evaluation with the EMA weights)."""
        model.load_state_dict(self.model.state_dict(), strict=False)
        return model


def build_ema(model, cfg, device):
    return EMA(model, cfg, device)
