"""One pre-LN decoder layer as a single autograd function over the sm_100a kernels.

Forward (7 kernels, tensor-parallel size 1):
  LN -> QKV GEMM(+bias) -> causal flash attention -> out-proj GEMM(+bias +residual)
  -> LN -> FC1 GEMM(+bias +ReLU) -> FC2 GEMM(+bias +residual)
Backward is written by hand: ReLU-backward and the residual-branch adds are folded into
GEMM / LayerNorm-backward epilogues, weight gradients are written straight into the FSDP
unit's flat gradient buffer when the parameters carry one.

The reference has this shape of code only for its sequence-parallel variant
(metaseq/modules/sequence_parallel_transformer_layer.py:92-387, no biases, non-affine
LN); the ordinary layer is a chain of autograd ops
(metaseq/modules/transformer_decoder_layer.py:263-284).  This function covers both:
biases and affine LayerNorm are optional, tensor parallelism reduces after the
row-parallel GEMMs (or, with ``sequence_parallel``, all-gathers before the
column-parallel GEMMs and reduce-scatters after the row-parallel ones), and
``recompute`` keeps only the layer input and redoes the forward during backward
(activation checkpointing, which the reference cannot combine with sequence parallel:
metaseq/models/transformer_lm.py:220-236).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.distributed as dist

from metaseq_b200.ops import functional as F
from metaseq_b200.ops.autograd import _direct_grad


@dataclass
class LayerSpec:
    B: int
    T: int
    heads_local: int
    head_dim: int
    scale: float
    eps: float
    tp_group: Any = None
    tp_world: int = 1
    sequence_parallel: bool = False
    recompute: bool = False
    comm: Any = None  # optional fused-communication provider (metaseq_b200.parallel.symm.TPComm)
    # dropout (training only): probability after out_proj / fc2, probability on the attention weights, and the
    # seeds of the three masks (drawn once per forward call, reused by recomputation and backward)
    dropout_p: float = 0.0
    attn_dropout_p: float = 0.0
    seeds: Any = None
    # attention beyond causality: per-token document starts ([B, T]) and per-head ALiBi slopes ([heads_local])
    doc_start: Any = None
    alibi_slopes: Any = None


def _all_reduce(t, spec):
    if spec.tp_world > 1:
        if spec.comm is not None:
            return spec.comm.all_reduce_(t)
        dist.all_reduce(t, group=spec.tp_group)
    return t


def _all_gather_rows(t, spec):
    if spec.tp_world == 1:
        return t
    if spec.comm is not None and hasattr(spec.comm, "all_gather_rows"):
        # peer push with arrival flags: the GEMM that reads the result as its A operand polls them per tile
        return spec.comm.all_gather_rows(t)
    out = torch.empty((t.shape[0] * spec.tp_world, t.shape[1]), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous(), group=spec.tp_group)
    return out


def _reduce_scatter_rows(t, spec):
    if spec.tp_world == 1:
        return t
    out = torch.empty((t.shape[0] // spec.tp_world, t.shape[1]), dtype=t.dtype, device=t.device)
    dist.reduce_scatter_tensor(out, t.contiguous(), group=spec.tp_group)
    return out


def _row_parallel_out(a, w, bias, residual, spec, seed=None):
    """``residual + dropout(bias + reduce(a @ w^T))`` over the tensor-parallel group (dropout when ``seed``)."""
    if seed is not None and spec.dropout_p > 0:
        if spec.tp_world == 1:
            part = F.gemm(a, w)
        elif spec.comm is not None:
            part = spec.comm.gemm_reduce_scatter(a, w) if spec.sequence_parallel else spec.comm.gemm_all_reduce(a, w)
        else:
            part = F.gemm(a, w)
            part = _reduce_scatter_rows(part, spec) if spec.sequence_parallel else _all_reduce(part, spec)
        return F.dropout_add(part, bias, residual, spec.dropout_p, seed)
    if spec.tp_world == 1:
        return F.gemm(a, w, bias=bias, residual=residual)
    if spec.comm is not None:
        if spec.sequence_parallel:
            return spec.comm.gemm_reduce_scatter(a, w, bias, residual)
        return spec.comm.gemm_all_reduce(a, w, bias, residual)
    part = F.gemm(a, w)
    if spec.sequence_parallel:
        part = _reduce_scatter_rows(part, spec)
    else:
        _all_reduce(part, spec)
    if bias is not None:
        part = part + bias
    return part.add_(residual)


def _dgrad_reduced(dy, w, spec: LayerSpec):
    """``reduce(dy @ w)`` over the tensor-parallel group: the input gradient of a column-parallel layer
    (all-reduce, or reduce-scatter along the sequence with sequence parallelism)."""
    if spec.tp_world > 1 and spec.comm is not None:
        if spec.sequence_parallel:
            return spec.comm.gemm_reduce_scatter(dy, w, None, None, b_mn=True)
        return spec.comm.gemm_all_reduce(dy, w, None, None, b_mn=True)
    d = F.gemm(dy, w, b_mn=True)
    return _reduce_scatter_rows(d, spec) if spec.sequence_parallel else _all_reduce(d, spec)


def _forward(x2, p, spec: LayerSpec):
    (ln1_w, ln1_b, qkv_w, qkv_b, out_w, out_b, ln2_w, ln2_b, fc1_w, fc1_b, fc2_w, fc2_b) = p
    B, T = spec.B, spec.T
    h1, mean1, rstd1 = F.layer_norm_fwd(x2, ln1_w, ln1_b, spec.eps)
    h1_full = _all_gather_rows(h1, spec) if spec.sequence_parallel else h1
    qkv = F.gemm(h1_full, qkv_w, bias=qkv_b)
    Dp = qkv.shape[1] // 3
    q3 = qkv.view(B, T, 3 * Dp)
    H, d = spec.heads_local, spec.head_dim
    k = q3[..., 0:Dp].view(B, T, H, d)
    v = q3[..., Dp:2 * Dp].view(B, T, H, d)
    q = q3[..., 2 * Dp:].view(B, T, H, d)
    s_attn, s_res1, s_res2 = spec.seeds if spec.seeds is not None else (None, None, None)
    ctx, lse = F.flash_attn_fwd(q, k, v, spec.scale, True, dropout_p=spec.attn_dropout_p if s_attn is not None else 0.0,
                                seed=s_attn or 0, doc_start=spec.doc_start, alibi_slopes=spec.alibi_slopes)
    ctx2 = ctx.view(B * T, Dp)
    x_mid = _row_parallel_out(ctx2, out_w, out_b, x2, spec, s_res1)
    h2, mean2, rstd2 = F.layer_norm_fwd(x_mid, ln2_w, ln2_b, spec.eps)
    h2_full = _all_gather_rows(h2, spec) if spec.sequence_parallel else h2
    act = F.gemm(h2_full, fc1_w, bias=fc1_b, relu=True)
    y = _row_parallel_out(act, fc2_w, fc2_b, x_mid, spec, s_res2)
    saved = (h1 if not spec.sequence_parallel else h1, mean1, rstd1, qkv, ctx, lse, x_mid, h2, mean2, rstd2, act)
    return y, saved


class FusedDecoderLayerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, spec: LayerSpec, *params):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y, saved = _forward(x2, params, spec)
        ctx.spec = spec
        ctx.params = params
        ctx.in_shape = shp
        if spec.recompute:
            ctx.save_for_backward(x2)
        else:
            ctx.save_for_backward(x2, *saved)
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy):
        spec: LayerSpec = ctx.spec
        params = ctx.params
        (ln1_w, ln1_b, qkv_w, qkv_b, out_w, out_b, ln2_w, ln2_b, fc1_w, fc1_b, fc2_w, fc2_b) = params
        if spec.recompute:
            (x2,) = ctx.saved_tensors
            with torch.no_grad():
                _, saved = _forward(x2, params, spec)
        else:
            x2, *saved = ctx.saved_tensors
        (h1, mean1, rstd1, qkv, attn, lse, x_mid, h2, mean2, rstd2, act) = saved
        B, T, H, d = spec.B, spec.T, spec.heads_local, spec.head_dim
        sp = spec.sequence_parallel
        dy2 = dy.reshape(x2.shape)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()

        def wgrad(param, a, b):
            # param.grad (+)= a^T @ b, a: [M, out], b: [M, in]
            return _direct_grad(param, lambda out, acc: F.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=acc))

        def bgrad(param, a):
            if param is None:
                return None
            return _direct_grad(param, lambda out, acc: F.colsum(a, out16=out, accumulate=acc))

        def ln_bwd(dyh, xin, mean, rstd, gw, gb, add):
            gv = getattr(gw, "_grad_view", None) if gw is not None else None
            if gv is not None:
                acc = getattr(gw, "_grad_filled", False)
                dx, _, _ = F.layer_norm_bwd(dyh, xin, mean, rstd, gw, add=add, dgamma_out=gv,
                                            dbeta_out=gb._grad_view, accumulate=acc)
                gw._grad_filled = True
                gb._grad_filled = True
                return dx, None, None
            return F.layer_norm_bwd(dyh, xin, mean, rstd, gw, add=add, need_param_grads=gw is not None)

        s_attn, s_res1, s_res2 = spec.seeds if spec.seeds is not None else (None, None, None)
        drop = spec.dropout_p > 0 and s_res2 is not None
        # ---- FC2 (row parallel): y = x_mid + dropout(b2 + reduce(act @ W2^T))
        dyb = F.dropout_add(dy2, None, None, spec.dropout_p, s_res2) if drop else dy2  # gradient of the dropped branch
        dy_full = _all_gather_rows(dyb, spec) if sp else dyb
        d_act = F.gemm(dy_full, fc2_w, b_mn=True, mask=act)  # ReLU backward fused
        g_fc2_w = wgrad(fc2_w, dy_full, act)
        g_fc2_b = bgrad(fc2_b, dyb)
        del dyb
        # ---- FC1 (column parallel)
        dh2 = _dgrad_reduced(d_act, fc1_w, spec)
        h2_full = _all_gather_rows(h2, spec) if sp else h2
        g_fc1_w = wgrad(fc1_w, d_act, h2_full)
        g_fc1_b = bgrad(fc1_b, d_act)
        del d_act, h2_full
        # ---- LN2 (+ residual branch gradient dy)
        dx_mid, g_ln2_w, g_ln2_b = ln_bwd(dh2, x_mid, mean2, rstd2, ln2_w, ln2_b, dy2)
        del dh2
        # ---- out_proj (row parallel)
        dxb = F.dropout_add(dx_mid, None, None, spec.dropout_p, s_res1) if (spec.dropout_p > 0 and s_res1 is not None) \
            else dx_mid
        dxm_full = _all_gather_rows(dxb, spec) if sp else dxb
        attn2 = attn.view(B * T, -1)
        d_attn = F.gemm(dxm_full, out_w, b_mn=True)
        g_out_w = wgrad(out_w, dxm_full, attn2)
        g_out_b = bgrad(out_b, dxb)
        del dxb
        # ---- attention
        Dp = qkv.shape[1] // 3
        dqkv = torch.empty_like(qkv)
        q3, dq3 = qkv.view(B, T, 3 * Dp), dqkv.view(B, T, 3 * Dp)
        sl = lambda t, i: t[..., i * Dp:(i + 1) * Dp].view(B, T, H, d)
        F.flash_attn_bwd(sl(q3, 2), sl(q3, 0), sl(q3, 1), attn, d_attn.view(B, T, Dp), lse, spec.scale, True,
                         sl(dq3, 2), sl(dq3, 0), sl(dq3, 1),
                         dropout_p=spec.attn_dropout_p if s_attn is not None else 0.0, seed=s_attn or 0,
                         doc_start=spec.doc_start, alibi_slopes=spec.alibi_slopes)
        del d_attn
        # ---- QKV (column parallel)
        dh1 = _dgrad_reduced(dqkv, qkv_w, spec)
        h1_full = _all_gather_rows(h1, spec) if sp else h1
        g_qkv_w = wgrad(qkv_w, dqkv, h1_full)
        g_qkv_b = bgrad(qkv_b, dqkv)
        del dqkv, h1_full
        # ---- LN1 (+ residual branch gradient dx_mid)
        dx, g_ln1_w, g_ln1_b = ln_bwd(dh1, x2, mean1, rstd1, ln1_w, ln1_b, dx_mid)
        hook = getattr(spec, "post_backward", None)
        return (dx.view(ctx.in_shape), None, g_ln1_w, g_ln1_b, g_qkv_w, g_qkv_b, g_out_w, g_out_b, g_ln2_w, g_ln2_b,
                g_fc1_w, g_fc1_b, g_fc2_w, g_fc2_b)


def fused_decoder_layer(x, spec: LayerSpec, ln1_w, ln1_b, qkv_w, qkv_b, out_w, out_b, ln2_w, ln2_b, fc1_w, fc1_b,
                        fc2_w, fc2_b):
    return FusedDecoderLayerFn.apply(x, spec, ln1_w, ln1_b, qkv_w, qkv_b, out_w, out_b, ln2_w, ln2_b, fc1_w, fc1_b,
                                     fc2_w, fc2_b)
