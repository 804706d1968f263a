"""Plain (non tensor-parallel) linear layer with optional on-device initialisation."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as TF

from metaseq_b200.ops import autograd as ops_ag
from metaseq_b200.ops import functional as ops_f


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, initialize_params_on_gpu: bool = False,
                 dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        device = torch.cuda.current_device() if (initialize_params_on_gpu and torch.cuda.is_available()) else None
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.in_features)
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, x):
        if ops_f.use_kernels(x) and x.dtype == self.weight.dtype:
            return ops_ag.linear(x, self.weight, self.bias)
        return TF.linear(x, self.weight, self.bias)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


def Embedding(num_embeddings, embedding_dim, padding_idx=None, initialize_params_on_gpu=False, dtype=None):
    device = torch.cuda.current_device() if (initialize_params_on_gpu and torch.cuda.is_available()) else None
    m = nn.Embedding(num_embeddings, embedding_dim, padding_idx=padding_idx, device=device, dtype=dtype)
    nn.init.normal_(m.weight, mean=0, std=embedding_dim ** -0.5)
    if padding_idx is not None:
        nn.init.constant_(m.weight[padding_idx], 0)
    return m
