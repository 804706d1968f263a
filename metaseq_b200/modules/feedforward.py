"""fc1 -> activation -> (dropout) -> fc2.  With tensor-parallel layers fc1 is column-parallel
and fc2 row-parallel (reference: metaseq/modules/feedforward.py)."""
from __future__ import annotations

import torch.nn as nn


class FeedForward(nn.Module):
    def __init__(self, fc1, activation_fn, fc2, dropout_module=None, model_parallel: bool = True):
        super().__init__()
        self.fc1, self.fc2 = fc1, fc2
        self.activation_fn = activation_fn
        self.dropout_module = dropout_module
        self.model_parallel = model_parallel

    def forward(self, x):
        h = self.fc1(x)
        if self.model_parallel:
            h = h[0]
        h = self.activation_fn(h)
        if self.dropout_module is not None:
            h = self.dropout_module(h)
        out = self.fc2(h)
        return out


def FeedForwardFn(x, fc1, activation_fn, fc2, dropout_module=None):
    """Functional form used by the decoder layer (fc2 returns ``(out, bias)`` when tensor parallel)."""
    h, _ = fc1(x)
    h = activation_fn(h)
    if dropout_module is not None:
        h = dropout_module(h)
    out, _ = fc2(h)
    return out
