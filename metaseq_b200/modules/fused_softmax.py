"""Stand-alone scale -> mask -> softmax over attention scores.

The reference exposes two autograd functions over its own softmax kernels
(metaseq/modules/megatron/model/fused_softmax.py:18-72): a causal one over ``[batch * heads, q, k]`` scores and a
masked one over ``[batch, heads, q, k]`` scores with a boolean ``[batch, 1, q, k]`` mask (true = hidden, filled with
-10000 after scaling).  The training and decoding paths of this package never materialise the score matrix: the
flash-attention kernels apply the causal bound, document starts and ALiBi slopes tile by tile.  These functions
keep the reference's interface for code that holds scores already (probing, analysis, custom layers); they save only
the probabilities for the backward pass, as the reference's kernels do, and compute in fp32 whatever the input type.
"""
from __future__ import annotations

import torch

_MASKED_FILL = -10000.0


def _softmax_backward(grad_out: torch.Tensor, probs: torch.Tensor, scale: float) -> torch.Tensor:
    g = grad_out.float() * probs.float()
    return ((g - probs.float() * g.sum(dim=-1, keepdim=True)) * scale).to(grad_out.dtype)


class ScaledUpperTriangMaskedSoftmax(torch.autograd.Function):
    """``softmax(scale * x)`` over keys ``<=`` the query index; hidden positions get probability exactly 0."""

    @staticmethod
    def forward(ctx, inputs: torch.Tensor, scale: float):
        assert inputs.dim() == 3, "expected [batch * heads, queries, keys]"
        q, k = inputs.shape[-2:]
        hidden = torch.ones(q, k, dtype=torch.bool, device=inputs.device).triu_(1)
        scores = (inputs.float() * scale).masked_fill_(hidden, float("-inf"))
        probs = torch.softmax(scores, dim=-1).to(inputs.dtype)
        ctx.save_for_backward(probs)
        ctx.scale = float(scale)
        return probs

    @staticmethod
    def backward(ctx, grad_out):
        (probs,) = ctx.saved_tensors
        return _softmax_backward(grad_out, probs, ctx.scale), None


class ScaledMaskedSoftmax(torch.autograd.Function):
    """``softmax(where(mask, -10000, scale * x))``: a fully hidden row comes out uniform, as in the reference."""

    @staticmethod
    def forward(ctx, inputs: torch.Tensor, mask: torch.Tensor, scale: float):
        assert inputs.dim() == 4, "expected [batch, heads, queries, keys]"
        scores = inputs.float() * scale
        if mask is not None:
            scores = scores.masked_fill(mask.to(torch.bool), _MASKED_FILL)
        probs = torch.softmax(scores, dim=-1).to(inputs.dtype)
        ctx.save_for_backward(probs)
        ctx.scale = float(scale)
        return probs

    @staticmethod
    def backward(ctx, grad_out):
        (probs,) = ctx.saved_tensors
        return _softmax_backward(grad_out, probs, ctx.scale), None, None


def scaled_upper_triang_masked_softmax(inputs: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    return ScaledUpperTriangMaskedSoftmax.apply(inputs, scale)


def scaled_masked_softmax(inputs: torch.Tensor, mask, scale: float = 1.0) -> torch.Tensor:
    return ScaledMaskedSoftmax.apply(inputs, mask, scale)
