"""Exponential moving average ("shadow") of a model's state.

Contract of the reference's ``EMA`` (metaseq/models/ema/ema.py:32-204): the shadow starts as a copy of the model
(or of ``--ema-seed-model``), ``step(model, updates)`` is called after every optimizer update, copies the model
while ``updates < --ema-start-update`` and afterwards moves the shadow by ``1 - decay`` towards it every
``--ema-update-freq`` updates; ``--ema-fp32`` keeps the running average in fp32 beside a 16-bit module;
``reverse`` loads the shadow into a model; the shadow's state dict travels in the checkpoint's extra state.

Here the average is advanced for all tensors at once with ``torch._foreach_*`` (two launches per update on a
GPU instead of two per tensor).  A fully sharded model is not deep-copied: the caller passes a second sharded
instance whose state already equals the trained model's, and the average runs over each rank's flat shards.
"""
from __future__ import annotations

import copy
import logging
from typing import Dict, Iterable, Optional

import torch

logger = logging.getLogger(__name__)


def load_ema_seed(path: str) -> Dict[str, torch.Tensor]:
    """Model state to start the shadow from: the ``ema`` entry of a checkpoint's extra state when it has one,
    its ``model`` entry otherwise."""
    from metaseq_b200 import checkpoint_utils

    state = checkpoint_utils.load_checkpoint_to_cpu(path)
    extra = state.get("extra_state") or {}
    return extra["ema"] if "ema" in extra else state["model"]


def _is_sharded(model) -> bool:
    return bool(getattr(model, "is_fsdp", False))


class EMA:
    def __init__(self, model, config, device=None, skip_keys: Optional[Iterable[str]] = None):
        self.config = config
        self.decay = config.ema_decay
        self.skip_keys = set(skip_keys or ())
        if _is_sharded(model):
            logger.info("EMA over a fully sharded model: using the given instance as the shadow (it must be a copy)")
            self.model = model
        else:
            self.model = copy.deepcopy(model)
        self.model.requires_grad_(False)
        seed = getattr(config, "ema_seed_model", None)
        if seed:
            self.model.load_state_dict(load_ema_seed(seed), strict=True)
        if device is not None:
            logger.info(f"Copying EMA model to device {device}")
            self.model = self.model.to(device=device)
        self.fp32_params: Dict[str, torch.Tensor] = {}
        if config.ema_fp32:
            self.build_fp32_params()
        self.update_freq_counter = 0

    # ----------------------------------------------------------------- access
    def get_model(self):
        return self.model

    def get_decay(self):
        return self.decay

    def _set_decay(self, decay):
        self.decay = decay

    # ------------------------------------------------------------ fp32 average
    def build_fp32_params(self, state_dict=None, device=None):
        """(Re)fills the fp32 running average from ``state_dict`` (default: the shadow module)."""
        if not self.config.ema_fp32:
            raise RuntimeError("the fp32 running average exists only with --ema-fp32")
        source = self.model.state_dict() if state_dict is None else state_dict
        for key, value in source.items():
            if not torch.is_tensor(value):
                continue
            held = self.fp32_params.get(key)
            if held is not None and held.shape == value.shape:
                held.copy_(value)
            else:
                self.fp32_params[key] = value.detach().float().clone() if value.is_floating_point() \
                    else value.detach().clone()
        if device is not None:
            self.fp32_params = {k: v.to(device) for k, v in self.fp32_params.items()}

    def restore(self, state_dict, build_fp32_params: bool = False):
        """Loads ``state_dict`` into the shadow module (and, on request, into the fp32 average)."""
        self.model.load_state_dict(state_dict, strict=False)
        if build_fp32_params:
            self.build_fp32_params(state_dict)

    # ------------------------------------------------------------------ update
    def _average_towards(self, live_state: Dict[str, torch.Tensor]):
        decay = float(self.decay)
        running = self.fp32_params if self.config.ema_fp32 else self.model.state_dict()
        result, avg, new = {}, [], []
        for key, value in live_state.items():
            if not torch.is_tensor(value):
                continue
            mine = running.get(key)
            if mine is None:  # a tensor the shadow has not seen yet starts at the live value
                mine = value.detach().float().clone() if (self.config.ema_fp32 and value.is_floating_point()) \
                    else value.detach().clone()
                if self.config.ema_fp32:
                    self.fp32_params[key] = mine
            if mine.shape != value.shape:
                raise ValueError(f"shape of {key} differs between model {tuple(value.shape)} and EMA "
                                 f"{tuple(mine.shape)}")
            result[key] = mine
            if "version" in key:
                continue  # format markers of modules are not averaged
            if key in self.skip_keys or not value.is_floating_point():
                mine.copy_(value)
            else:
                avg.append(mine)
                new.append(value.detach().to(device=mine.device, dtype=mine.dtype))
        if avg:
            torch._foreach_mul_(avg, decay)
            torch._foreach_add_(avg, new, alpha=1.0 - decay)
        # write back: a no-op copy where ``running`` aliases the module, a cast where the average is fp32, a reload
        # of the flat shards for a sharded shadow
        self.model.load_state_dict(result, strict=False)

    def _step_internal(self, new_model, updates=None):
        with torch.no_grad():
            self._average_towards(new_model.state_dict())

    def step(self, new_model, updates=None):
        """Once per optimizer update.  Before ``ema_start_update`` the decay is 0 (the shadow copies the model)."""
        starting = updates is not None and updates < self.config.ema_start_update
        self._set_decay(0 if starting else self.config.ema_decay)
        if updates is not None and self.config.ema_update_freq > 1:
            self.update_freq_counter += 1
            if self.update_freq_counter < self.config.ema_update_freq:
                return
            self.update_freq_counter = 0
        self._step_internal(new_model, updates)

    def reverse(self, model):
        """Loads the averaged parameters into ``model`` (evaluation or fine-tuning from the shadow)."""
        model.load_state_dict(self.model.state_dict(), strict=False)
        return model


def build_ema(model, cfg, device):
    return EMA(model, cfg, device)
