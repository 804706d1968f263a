"""Dropout that can stay active at inference when asked to (retain_dropout)."""
from __future__ import annotations

import logging
from typing import List, Optional

import torch.nn as nn
import torch.nn.functional as TF

logger = logging.getLogger(__name__)


class Dropout(nn.Module):
    def __init__(self, p, module_name=None):
        super().__init__()
        self.p = p
        self.module_name = module_name
        self.apply_during_inference = False

    def extra_repr(self):
        return f"p={self.p}"

    def forward(self, x, inplace: bool = False):
        if self.p > 0 and (self.training or self.apply_during_inference):
            return TF.dropout(x, p=self.p, training=True, inplace=inplace)
        return x

    def make_generation_fast_(self, name: str, retain_dropout: bool = False,
                              retain_dropout_modules: Optional[List[str]] = None, **kwargs):
        if retain_dropout:
            if retain_dropout_modules is None or self.module_name in retain_dropout_modules:
                logger.info(f"Enabling dropout during inference for module: {name}")
                self.apply_during_inference = True
