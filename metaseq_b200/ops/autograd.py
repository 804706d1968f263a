"""Autograd wrappers over the raw operators in ``functional``.

These make the kernels usable from ordinary ``nn.Module`` code (the modular
tensor-parallel layers, the output projection, the criterions).  The fused
decoder layer (``metaseq_b200.modules.fused_layer``) calls the raw operators
directly instead, with its own hand-written backward.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import functional as F


def _direct_grad(param: Optional[torch.Tensor], compute, shape_like: Optional[torch.Tensor] = None):
    """Gradient for a parameter.  When the parameter carries a ``_grad_view`` (a slice of an
    FSDP unit's flat gradient buffer) the gradient is written or accumulated there and
    ``None`` is returned to autograd; otherwise a fresh tensor is returned."""
    if param is None:
        return None
    view = getattr(param, "_grad_view", None)
    if view is None:
        return compute(None, False)
    filled = getattr(param, "_grad_filled", False)
    compute(view, filled)
    param._grad_filled = True
    return None


_UPSTREAM_GRAD_HINT = [None]


def set_upstream_grad_hint(value: Optional[float]):
    """The factor that the backward pass is expected to bring to the loss (the fp16 optimizer's loss scale), told to
    the loss kernels before the forward pass: they store their gradient already multiplied by it, and the backward
    pass rescales only where the factor that really arrives differs.  ``None`` (or 1) switches the guess off."""
    _UPSTREAM_GRAD_HINT[0] = float(value) if value else None


def upstream_grad_hint() -> float:
    v = _UPSTREAM_GRAD_HINT[0]
    return v if (v is not None and v > 0 and v == v and v != float("inf")) else 1.0


class LinearFn(torch.autograd.Function):
    """``y = act(x @ W^T + b) + residual`` with the epilogue fused into the GEMM.  ``stats_out`` (a dict) asks for
    the per-tile softmax pieces of every output row (``functional.gemm_with_row_stats``) under ``"row_stats"``."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, relu: bool, stats_out=None):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        res2 = residual.reshape(-1, weight.shape[0]) if residual is not None else None
        if stats_out is not None and res2 is None and not relu:
            y, stats_out["row_stats"] = F.gemm_with_row_stats(x2, weight, bias)
        else:
            y = F.gemm(x2, weight, bias=bias, residual=res2, relu=relu)
        ctx.relu = relu
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.params = (weight, bias)
        ctx.save_for_backward(x2, weight, y if relu else None)
        ctx.in_shape = shp
        return y.view(*shp[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight, y = ctx.saved_tensors
        wparam, bparam = ctx.params
        dy2 = dy.reshape(-1, weight.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.relu:
            if ctx.has_res:
                raise RuntimeError("relu with a residual is not differentiable through the fused epilogue")
            dz = dy2 * (y > 0).to(dy2.dtype)
        else:
            dz = dy2
        dx = F.gemm(dz, weight, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _direct_grad(wparam, lambda out, acc: F.gemm(dz, x2, a_mn=True, b_mn=True, out=out, accumulate=acc))
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _direct_grad(bparam, lambda out, acc: F.colsum(dz, out16=out, accumulate=acc))
        dres = dy if ctx.has_res else None
        return (dx.view(ctx.in_shape) if dx is not None else None), dw, db, dres, None, None


def linear(x, weight, bias=None, residual=None, relu: bool = False, row_stats: bool = False):
    """With ``row_stats`` the result carries ``_msq_row_stats``: the ``(max, sum-exp)`` tables per column tile that
    a cross entropy over the same rows can start from (``None`` where the kernel did not produce them)."""
    if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
        if row_stats:
            holder = {}
            y = LinearFn.apply(x, weight, bias, residual, relu, holder)
            y._msq_row_stats = holder.get("row_stats")
            return y
        return LinearFn.apply(x, weight, bias, residual, relu)
    shp = x.shape
    res2 = residual.reshape(-1, weight.shape[0]) if residual is not None else None
    y = F.gemm(x.reshape(-1, shp[-1]), weight, bias=bias, residual=res2, relu=relu)
    return y.view(*shp[:-1], weight.shape[0])


class LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps: float):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        y, mean, rstd = F.layer_norm_fwd(x2, gamma, beta, eps)
        ctx.save_for_backward(x2, mean, rstd, gamma)
        ctx.params = (gamma, beta)
        ctx.in_shape = shp
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, mean, rstd, gamma = ctx.saved_tensors
        gparam, bparam = ctx.params
        dy2 = dy.reshape(x2.shape).contiguous()
        gv = getattr(gparam, "_grad_view", None) if gparam is not None else None
        if gv is not None:
            acc = getattr(gparam, "_grad_filled", False)
            dx, _, _ = F.layer_norm_bwd(dy2, x2, mean, rstd, gamma, dgamma_out=gv,
                                        dbeta_out=bparam._grad_view, accumulate=acc)
            gparam._grad_filled = True
            bparam._grad_filled = True
            return dx.view(ctx.in_shape), None, None, None
        dx, dg, db = F.layer_norm_bwd(dy2, x2, mean, rstd, gamma, need_param_grads=gamma is not None)
        return dx.view(ctx.in_shape), dg, db, None


class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, eps: float):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        y, rstd = F.rms_norm_fwd(x2, gamma, eps)
        ctx.save_for_backward(x2, rstd, gamma)
        ctx.in_shape = shp
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, rstd, gamma = ctx.saved_tensors
        dx, dg = F.rms_norm_bwd(dy.reshape(x2.shape).contiguous(), x2, rstd, gamma)
        return dx.view(ctx.in_shape), dg, None


def rms_norm(x, gamma, eps: float = 1e-5):
    return RMSNormFn.apply(x, gamma, eps)


def layer_norm(x, gamma, beta, eps: float = 1e-5):
    return LayerNormFn.apply(x, gamma, beta, eps)


class FlashAttnFn(torch.autograd.Function):
    """Causal attention over a packed ``[B, T, 3*H*d]`` projection laid out as (k | v | q)."""

    @staticmethod
    def forward(ctx, qkv, num_heads: int, scale: float, causal: bool, doc_start=None, alibi_slopes=None):
        B, T, W = qkv.shape
        D = W // 3
        d = D // num_heads
        k = qkv[..., 0:D].view(B, T, num_heads, d)
        v = qkv[..., D:2 * D].view(B, T, num_heads, d)
        q = qkv[..., 2 * D:].view(B, T, num_heads, d)
        out, lse = F.flash_attn_fwd(q, k, v, scale, causal, doc_start=doc_start, alibi_slopes=alibi_slopes)
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (num_heads, scale, causal)
        ctx.masks = (doc_start, alibi_slopes)  # integer / constant tensors: no gradient flows to them
        return out

    @staticmethod
    def backward(ctx, d_out):
        qkv, out, lse = ctx.saved_tensors
        H, scale, causal = ctx.meta
        B, T, W = qkv.shape
        D = W // 3
        d = D // H
        dqkv = torch.empty_like(qkv)
        views = lambda t: (t[..., 0:D].view(B, T, H, d), t[..., D:2 * D].view(B, T, H, d), t[..., 2 * D:].view(B, T, H, d))
        k, v, q = views(qkv)
        dk, dv, dq = views(dqkv)
        F.flash_attn_bwd(q, k, v, out, d_out.contiguous(), lse, scale, causal, dq, dk, dv, doc_start=ctx.masks[0],
                         alibi_slopes=ctx.masks[1])
        return dqkv, None, None, None, None, None


def flash_attention_packed(qkv, num_heads: int, scale: float, causal: bool = True, doc_start=None, alibi_slopes=None):
    """``doc_start`` (``[B, T]``) / ``alibi_slopes`` (``[H]``): see ``functional.flash_attn_fwd``."""
    return FlashAttnFn.apply(qkv, num_heads, scale, causal, doc_start, alibi_slopes)


class CrossEntropyFn(torch.autograd.Function):
    """Summed NLL over rows.  The forward overwrites the logits with the gradient
    ``(softmax - onehot) * grad_scale``; the backward only rescales it by the incoming
    gradient (1 in the usual ``loss.backward()``), so fp32 logits are never materialised."""

    @staticmethod
    def forward(ctx, logits, target, ignore_index: int, row_stats=None):
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        ctx.pre_scaled = upstream_grad_hint()
        if row_stats is not None:
            loss_rows = F.cross_entropy_from_row_stats(l2, target.reshape(-1), ignore_index, ctx.pre_scaled, row_stats)
        else:
            loss_rows, _ = F.cross_entropy_fwd_bwd(l2, target.reshape(-1), ignore_index, ctx.pre_scaled, True)
        ctx.save_for_backward(l2)
        ctx.shape = logits.shape
        return loss_rows.sum()

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        # g is the scalar d(total)/d(loss), typically the loss scale, which the forward pass already applied when it
        # was announced (set_upstream_grad_hint): then nothing is left to do
        if g.numel() == 1:
            F.scale_rows_(grad, g, ref=ctx.pre_scaled)  # in place: the saved tensor is the consumed logits buffer
        return grad.view(ctx.shape), None, None, None


def cross_entropy_sum(logits, target, ignore_index: int):
    """``logits`` is consumed (overwritten in place).  Logits that carry ``_msq_row_stats`` (``linear(...,
    row_stats=True)``) skip the pass that finds the row maxima and sums."""
    return CrossEntropyFn.apply(logits, target, ignore_index, getattr(logits, "_msq_row_stats", None))


class EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, positions, tok_w, pos_w, scale: float, pad_idx: int, vocab_start: int):
        ctx.save_for_backward(tokens, positions)
        ctx.params = (tok_w, pos_w)
        ctx.meta = (scale, pad_idx, vocab_start, tok_w.shape[0], pos_w.shape[0] if pos_w is not None else 0)
        return F.embed_fwd(tokens, positions, tok_w, pos_w, scale, vocab_start=vocab_start)

    @staticmethod
    def backward(ctx, dy):
        tokens, positions = ctx.saved_tensors
        tok_w, pos_w = ctx.params
        scale, pad_idx, vstart, nt, np_ = ctx.meta
        dtok32, dpos32 = F.embed_bwd(tokens, positions, dy.contiguous(), nt, np_, scale, pad_idx, vocab_start=vstart,
                                     need_pos=pos_w is not None)

        def fold(src32, param):
            def compute(out, acc):
                if out is None:
                    return src32.to(param.dtype)
                return F.fold_fp32_into(src32, out, acc)
            return _direct_grad(param, compute)

        dt = fold(dtok32, tok_w)
        dp = fold(dpos32, pos_w) if pos_w is not None else None
        return None, None, dt, dp, None, None, None


def embedding(tokens, positions, tok_w, pos_w, scale: float, pad_idx: int, vocab_start: int = 0):
    return EmbeddingFn.apply(tokens, positions, tok_w, pos_w, scale, pad_idx, vocab_start)
