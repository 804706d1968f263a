"""Activation helpers: gelu / relu with explicit backward forms (used by hand-written
layer backward passes) and the gated variants swiglu / geglu
(reference: metaseq/modules/activation_functions.py)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as TF


def gelu(x: torch.Tensor) -> torch.Tensor:
    return x * 0.5 * (1.0 + torch.tanh(0.79788456 * x * (1 + 0.044715 * x * x)))


def gelu_back(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    t = torch.tanh(0.79788456 * x * (1 + 0.044715 * x * x))
    ff = 0.5 * x * ((1 - t * t) * (0.79788456 + 0.1070322243 * x * x)) + 0.5 * (1 + t)
    return ff * g


def relu(x: torch.Tensor) -> torch.Tensor:
    return TF.relu(x)


def relu_back(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    return g.masked_fill(x <= 0, 0)


def swiglu(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    return TF.silu(x) * gate


def geglu(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    return TF.gelu(x) * gate


class GatedActivation(nn.Module):
    """Splits the last dimension in two and gates one half with the other."""

    def __init__(self, kind: str):
        super().__init__()
        assert kind in ("swiglu", "geglu")
        self.kind = kind

    def forward(self, x):
        a, b = x.chunk(2, dim=-1)
        return swiglu(a, b) if self.kind == "swiglu" else geglu(a, b)


class ActivationFn(nn.Module):
    def __init__(self, name, fc1_builder, embed_dim, ffn_dim, **fc1_kwargs):
        super().__init__()
        self.fn = self.__get_fn(name)
        self.gate = None
        if self.__is_gated(name):
            self.gate = fc1_builder(embed_dim, ffn_dim, **fc1_kwargs)

    def forward(self, fc1_in, fc1_out, model_parallel=False):
        if self.gate is not None:
            g = self.gate(fc1_in)
            if model_parallel:
                g = g[0]
            return self.fn(fc1_out, g)
        return self.fn(fc1_out)

    @staticmethod
    def __get_fn(name):
        from metaseq_b200 import utils

        if name == "swiglu":
            return swiglu
        if name == "geglu":
            return geglu
        return utils.get_activation_fn(name)

    @staticmethod
    def __is_gated(name):
        return name in ("swiglu", "geglu")
