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
