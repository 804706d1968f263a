"""LayerNorm factory.  On a GPU with 16-bit activations the forward and backward run the
sm_100a LayerNorm kernels; elsewhere ``torch.nn.functional.layer_norm``.  (The reference
picks apex FusedLayerNorm when importable: metaseq/modules/layer_norm.py:10-33.)"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as TF

from metaseq_b200.ops import autograd as ops_ag
from metaseq_b200.ops import functional as ops_f


class FusedLayerNorm(nn.LayerNorm):
    def forward(self, x):
        if ops_f.use_kernels(x) and x.shape[-1] % 8 == 0 and (self.weight is None or self.weight.dtype == x.dtype):
            return ops_ag.layer_norm(x, self.weight, self.bias, self.eps)
        return TF.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)


def LayerNorm(normalized_shape, eps=1e-5, elementwise_affine=True, export=False):
    return FusedLayerNorm(normalized_shape, eps, elementwise_affine)


class RMSNorm(nn.Module):
    """``x * rsqrt(mean(x^2) + eps) * weight``: the LayerNorm kernels without centring and shift (the reference's
    fused LayerNorm extension exports the same as ``rms_forward_affine`` / ``rms_backward_affine``:
    metaseq/modules/apex/layer_norm_cuda.cpp:459-471; no Python module of the reference uses them)."""

    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True):
        super().__init__()
        dim = normalized_shape if isinstance(normalized_shape, int) else normalized_shape[-1]
        self.normalized_shape = (dim,)
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim)) if elementwise_affine else None

    def forward(self, x):
        w = self.weight
        if w is not None and w.dtype != x.dtype:
            w = w.to(x.dtype)
        return ops_ag.rms_norm(x, w, self.eps)


class LayerNormFp32(nn.LayerNorm):
    """LayerNorm computed in fp32 regardless of the input dtype."""

    def forward(self, x):
        out = TF.layer_norm(x.float(), self.normalized_shape,
                            self.weight.float() if self.weight is not None else None,
                            self.bias.float() if self.bias is not None else None, self.eps)
        return out.type_as(x)


class GroupNormFp32(nn.GroupNorm):
    def forward(self, x):
        out = TF.group_norm(x.float(), self.num_groups,
                            self.weight.float() if self.weight is not None else None,
                            self.bias.float() if self.bias is not None else None, self.eps)
        return out.type_as(x)
