"""Dropout layer that knows its owner's name, so that generation can be told to keep some dropout layers active
(``retain_dropout`` / ``retain_dropout_modules`` of ``make_generation_fast_``; reference: metaseq/modules/dropout.py)."""
from __future__ import annotations

import logging
from typing import List, Optional

import torch.nn as nn
import torch.nn.functional as TF

logger = logging.getLogger(__name__)


class Dropout(nn.Module):
    """``p``: drop probability.  ``module_name``: the class name of the module that owns this layer; it is what
    ``retain_dropout_modules`` is matched against."""

    def __init__(self, p, module_name=None):
        super().__init__()
        self.p, self.module_name = p, module_name
        self.apply_during_inference = False  # switched on by make_generation_fast_

    @property
    def active(self) -> bool:
        return self.p > 0 and (self.training or self.apply_during_inference)

    def forward(self, x, inplace: bool = False):
        return TF.dropout(x, p=self.p, training=True, inplace=inplace) if self.active else x

    def make_generation_fast_(self, name: str, retain_dropout: bool = False,
                              retain_dropout_modules: Optional[List[str]] = None, **kwargs):
        wanted = retain_dropout and (retain_dropout_modules is None or self.module_name in retain_dropout_modules)
        if wanted:
            self.apply_during_inference = True
            logger.info(f"Enabling dropout during inference for module: {name}")

    def extra_repr(self):
        return f"p={self.p}"
