"""Tensor-parallel multi-head self-attention with a fused (k | v | q) projection.

Contract kept from the reference (metaseq/modules/multihead_attention.py:42-577):
the fused projection's output columns are ordered K, V, Q within each
tensor-parallel partition (:316-319); ``out_proj`` is row-parallel with
``skip_bias_add`` so its bias is added by the layer after the reduction
(:256-265); inference keeps a key/value cache in ``incremental_state``.

Differences by design: activations are batch-first ``[B, T, D]``; the training
path is one causal flash-attention kernel instead of baddbmm + masked-softmax
kernel + bmm; the cache is preallocated to ``max_positions`` and appended in
place rather than re-concatenated every token.
"""
from __future__ import annotations

import math
import uuid
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as TF

from metaseq_b200 import utils
from metaseq_b200.modules.attention_bias import AttentionBias
from metaseq_b200.modules.dropout import Dropout
from metaseq_b200.ops import autograd as ops_ag
from metaseq_b200.ops import functional as ops_f
from metaseq_b200.parallel import mpu
from metaseq_b200.parallel.layers import ColumnParallelLinear, RowParallelLinear


class KVCache:
    """Preallocated per-layer cache: ``k``/``v`` are ``[B, Tmax, H_local * d]``; ``length`` counts
    the positions already filled."""

    def __init__(self, bsz: int, max_len: int, width: int, dtype, device):
        self.k = torch.zeros(bsz, max_len, width, dtype=dtype, device=device)
        self.v = torch.zeros(bsz, max_len, width, dtype=dtype, device=device)
        self.length = 0

    def append(self, k_new, v_new):
        n = k_new.shape[1]
        end = self.length + n
        if end > self.k.shape[1]:
            grow = max(end, 2 * self.k.shape[1])
            for name in ("k", "v"):
                old = getattr(self, name)
                buf = torch.zeros(old.shape[0], grow, old.shape[2], dtype=old.dtype, device=old.device)
                buf[:, : self.length] = old[:, : self.length]
                setattr(self, name, buf)
        self.k[:, self.length:end] = k_new
        self.v[:, self.length:end] = v_new
        self.length = end

    def reorder(self, new_order):
        self.k = self.k.index_select(0, new_order)
        self.v = self.v.index_select(0, new_order)


class ModelParallelMultiheadAttention(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True,
                 use_cpu_initialization: bool = True, full_megatron_init: bool = False,
                 full_megatron_init_scalar: float = 1.0, megatron_init_sigma: Optional[float] = None,
                 num_layers: Optional[int] = None, dtype=None, device=None, sequence_parallel: bool = False,
                 truncate_init: bool = False, max_positions: int = 2048, kdim: Optional[int] = None,
                 vdim: Optional[int] = None, self_attention: bool = True, attn_variant=None, xf_attn_op=None):
        super().__init__()
        # arguments of the reference's constructor that have one admissible value here: keys and values come from
        # the same input as the queries, and the attention kernel is not selectable
        assert self_attention and kdim in (None, embed_dim) and vdim in (None, embed_dim), \
            "only self-attention over inputs of the model width is built"
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.head_dim = embed_dim // num_heads
        assert self.head_dim * num_heads == embed_dim, "embed_dim must be divisible by num_heads"
        self.model_parallel_size = mpu.get_tensor_model_parallel_world_size()
        self.num_heads_partition = mpu.divide(num_heads, self.model_parallel_size)
        self.scaling = self.head_dim ** -0.5
        self.dropout_module = Dropout(dropout, module_name=self.__class__.__name__)
        self.sequence_parallel = sequence_parallel
        self.inference = False
        self.max_positions = max_positions
        self._cache_key = str(uuid.uuid4())

        if full_megatron_init:
            assert megatron_init_sigma is not None
            init_w = utils.init_method_normal(megatron_init_sigma * full_megatron_init_scalar)
            init_o = utils.scaled_init_method_normal(megatron_init_sigma * full_megatron_init_scalar, num_layers)
        else:
            # each of k, v, q initialised like a separate [D, D] projection with gain 1/sqrt(2)
            def init_w(w):
                d0 = w.shape[0] // 3
                for i in range(3):
                    nn.init.xavier_uniform_(w[i * d0:(i + 1) * d0], gain=1 / math.sqrt(2))
                return w

            init_o = nn.init.xavier_uniform_
        self.qkv_proj = ColumnParallelLinear(
            embed_dim, 3 * embed_dim, bias=bias, gather_output=False, init_method=init_w, stride=3,
            use_cpu_initialization=use_cpu_initialization, dtype=dtype, device=device,
            sequence_parallel=sequence_parallel)
        self.out_proj = RowParallelLinear(
            embed_dim, embed_dim, bias=bias, input_is_parallel=True, init_method=init_o, skip_bias_add=True,
            use_cpu_initialization=use_cpu_initialization, dtype=dtype, device=device,
            sequence_parallel=sequence_parallel)

    # ------------------------------------------------------------------ cache
    def _get_cache(self, incremental_state) -> Optional[KVCache]:
        return incremental_state.get(self._cache_key) if incremental_state is not None else None

    def reorder_incremental_state(self, incremental_state, new_order):
        c = self._get_cache(incremental_state)
        if c is not None:
            c.reorder(new_order)
        return incremental_state

    # ---------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, bt: Tuple[int, int], incremental_state: Optional[Dict] = None,
                key_padding_mask: Optional[torch.Tensor] = None, attn_mask: Optional[torch.Tensor] = None):
        """``x``: ``[B, T, D]`` (or ``[B*T/p, D]`` under sequence parallelism); returns
        ``(out, out_proj_bias)`` with the bias not yet added."""
        B, T = bt
        qkv, _ = self.qkv_proj(x)  # [..., 3 * D / p] as (k | v | q)
        qkv = qkv.reshape(B, T, -1)
        Dp = qkv.shape[-1] // 3
        H, d = self.num_heads_partition, self.head_dim
        cache = self._get_cache(incremental_state)
        use_cache = incremental_state is not None

        structured = attn_mask if isinstance(attn_mask, AttentionBias) else None
        if not use_cache and key_padding_mask is None and (attn_mask is None or structured is not None) \
                and self.dropout_module.p == 0.0 and ops_f.use_kernels(qkv) and ops_f.attn_head_dim_ok(d):
            ctx = ops_ag.flash_attention_packed(qkv.contiguous(), H, self.scaling, True,
                                                structured.doc_start if structured is not None else None,
                                                structured.slopes if structured is not None else None)
        else:
            k = qkv[..., 0:Dp]
            v = qkv[..., Dp:2 * Dp]
            q = qkv[..., 2 * Dp:]
            past = 0
            if use_cache:
                if cache is None:
                    cache = KVCache(B, max(self.max_positions + 2, T), Dp, qkv.dtype, qkv.device)
                    incremental_state[self._cache_key] = cache
                past = cache.length
                cache.append(k, v)
                if T == 1 and attn_mask is None and not self.training and ops_f.use_kernels(q) \
                        and ops_f.decode_head_dim_ok(self.head_dim):
                    # one generated token: a single kernel streams the preallocated cache once
                    ctx = ops_f.decode_attn(q, cache.k, cache.v, cache.length, self.num_heads_partition, self.scaling,
                                            key_padding_mask)
                    out, bias = self.out_proj(ctx)
                    return out, bias
                k = cache.k[:, : cache.length]
                v = cache.v[:, : cache.length]
            if structured is not None:  # the PyTorch paths below take the additive mask (causality included)
                attn_mask = structured.dense(T, k.shape[1], past, q.device)
            ctx = self._attend(q, k, v, B, T, past, key_padding_mask, attn_mask)  # cached or masked path
        if self.sequence_parallel:
            ctx = ctx.reshape(B * T, -1)
        out, bias = self.out_proj(ctx)
        return out, bias

    def _attend(self, q, k, v, B, T, past, key_padding_mask, attn_mask):
        H, d = self.num_heads_partition, self.head_dim
        S = k.shape[1]
        if past == 0 and T == S and key_padding_mask is None and attn_mask is None and not self.training \
                and ops_f.use_kernels(q) and ops_f.attn_head_dim_ok(d):
            out, _ = ops_f.flash_attn_fwd(q.reshape(B, T, H, d), k.reshape(B, S, H, d), v.reshape(B, S, H, d),
                                          self.scaling, True)
            return out
        if q.is_cuda and past == 0 and T == S and key_padding_mask is None and attn_mask is None and \
                q.dtype in (torch.float16, torch.bfloat16) and not (self.training and self.dropout_module.p > 0):
            # library attention (PyTorch SDPA): only reached with the "torch" operator backend, where it
            # stands in for the baseline without materialising [T, T] scores
            o = TF.scaled_dot_product_attention(
                q.reshape(B, T, H, d).transpose(1, 2), k.reshape(B, S, H, d).transpose(1, 2),
                v.reshape(B, S, H, d).transpose(1, 2), is_causal=True, scale=self.scaling)
            return o.transpose(1, 2).reshape(B, T, H * d)
        qh = q.reshape(B, T, H, d).transpose(1, 2).float() * self.scaling
        kh = k.reshape(B, S, H, d).transpose(1, 2).float()
        vh = v.reshape(B, S, H, d).transpose(1, 2)
        scores = torch.matmul(qh, kh.transpose(-1, -2))  # [B, H, T, S]
        if attn_mask is not None:
            scores = scores + attn_mask.float()
        else:
            # query i (absolute position past + i) sees keys 0..past+i
            qpos = torch.arange(past, past + T, device=q.device)[:, None]
            kpos = torch.arange(S, device=q.device)[None, :]
            scores = scores.masked_fill(kpos > qpos, float("-inf"))
        if key_padding_mask is not None:
            scores = scores.masked_fill(key_padding_mask[:, None, None, :S].bool(), float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        if self.training and self.dropout_module.p > 0:
            with mpu.get_cuda_rng_tracker().fork():
                probs = self.dropout_module(probs)
        ctx = torch.matmul(probs.to(vh.dtype), vh)  # [B, H, T, d]
        return ctx.transpose(1, 2).reshape(B, T, H * d)

    def make_generation_fast_(self, **kwargs):
        self.inference = True
