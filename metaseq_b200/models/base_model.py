"""Model base classes (reference: metaseq/models/base_model.py:93-135 for
``make_generation_fast_``)."""
from __future__ import annotations

import logging
from argparse import Namespace
from typing import Dict, Optional

import torch
import torch.nn as nn

from metaseq_b200.dataclass.utils import gen_parser_from_dataclass

logger = logging.getLogger(__name__)


def check_type(module, expected_type):
    """Asserts the type of a module, looking through a sharding wrapper."""
    inner = getattr(module, "unwrapped_module", module)
    assert isinstance(inner, expected_type), f"{type(inner)} != {expected_type}"


class BaseModel(nn.Module):
    """Decoder-only model: ``forward(src_tokens) -> (logits [B, T, V], extra)``.  ``BaseModel(decoder)`` is the
    reference's constructor (metaseq/models/base_model.py:33-41); a subclass that builds its decoder later may
    call it without one."""

    def __init__(self, decoder=None):
        super().__init__()
        self._is_generation_fast = False
        if decoder is not None:
            from .base_decoder import BaseDecoder

            check_type(decoder, BaseDecoder)
            self.decoder = decoder

    @classmethod
    def from_pretrained(cls, model_name_or_path, checkpoint_file="model.pt", data_name_or_path=".",
                        skip_prepare_for_inference=False, **kwargs):
        """The reference leaves this unimplemented as well (metaseq/models/base_model.py:137-146): released
        checkpoints are loaded through ``hub_utils.GeneratorInterface`` or ``checkpoint_utils``."""
        raise NotImplementedError

    @classmethod
    def hub_models(cls):
        return {}

    def forward(self, src_tokens, **kwargs):
        return self.decoder(src_tokens, **kwargs)

    def forward_decoder(self, prev_output_tokens, **kwargs):
        return self.decoder(prev_output_tokens, **kwargs)

    def extract_features(self, src_tokens, **kwargs):
        return self.decoder.extract_features(src_tokens, **kwargs)

    def output_layer(self, features, **kwargs):
        return self.decoder.output_layer(features, **kwargs)

    def max_decoder_positions(self):
        return self.decoder.max_positions()

    @property
    def supported_targets(self):
        return {"future"}

    @classmethod
    def add_args(cls, parser):
        dc = getattr(cls, "__dataclass", None)
        if dc is not None:
            gen_parser_from_dataclass(parser, dc(), delete_default=True)

    @classmethod
    def build_model(cls, args, task):
        raise NotImplementedError("Model must implement the build_model method")

    def get_targets(self, sample, net_output):
        return sample["target"]

    def get_normalized_probs(self, net_output, log_probs: bool, sample=None):
        logits = net_output[0] if isinstance(net_output, (tuple, list)) else net_output
        return self.decoder.get_normalized_probs(logits, log_probs, sample)

    def max_positions(self):
        dec = getattr(self, "decoder", None)
        return dec.max_positions() if dec is not None else None

    def load_state_dict(self, state_dict, strict=True, model_cfg=None):
        self.upgrade_state_dict(state_dict)
        return super().load_state_dict(state_dict, strict)

    def upgrade_state_dict(self, state_dict):
        self.upgrade_state_dict_named(state_dict, "")

    def upgrade_state_dict_named(self, state_dict, name):
        def walk(m, prefix):
            if len(prefix) > 0:
                prefix += "."
            for n, c in m.named_children():
                cname = prefix + n
                if hasattr(c, "upgrade_state_dict_named"):
                    c.upgrade_state_dict_named(state_dict, cname)
                elif hasattr(c, "upgrade_state_dict"):
                    c.upgrade_state_dict(state_dict)
                walk(c, cname)

        walk(self, name)

    def set_num_updates(self, num_updates):
        for m in self.modules():
            if hasattr(m, "set_num_updates") and m is not self:
                m.set_num_updates(num_updates)

    def prepare_for_inference_(self, cfg):
        kwargs = {}
        if getattr(cfg.generation, "retain_dropout", False):
            kwargs["retain_dropout"] = True
        self.make_generation_fast_(**kwargs)

    def make_generation_fast_(self, **kwargs):
        """Freezes the model for generation: switches attention to the cached inference path,
        puts modules in eval mode and makes a later ``train()`` an error."""
        if self._is_generation_fast:
            return
        self._is_generation_fast = True

        def apply_fast(module, prefix):
            if len(prefix) > 0:
                prefix += "."
            seen = set()
            for n, m in module.named_modules():
                if m is not module and hasattr(m, "make_generation_fast_") and m not in seen and \
                        not isinstance(m, BaseModel):
                    seen.add(m)
                    m.make_generation_fast_(name=prefix + n, **kwargs)

        apply_fast(self, "")
        self.eval()

        def train(mode=True):
            if mode:
                raise RuntimeError("cannot train after make_generation_fast")
            return self  # .eval() keeps returning the module

        self.train = train


class LanguageModel(BaseModel):
    """Kept as the name that this package's models derive from; everything lives in ``BaseModel``."""

    def __init__(self, decoder):
        super().__init__(decoder)
