"""Pre-LN transformer decoder block (self-attention + feed-forward), tensor parallel.

Parameter names and registration order are part of the checkpoint contract
(flat-parameter order inside an FSDP unit):
``self_attn.qkv_proj.{weight,bias}``, ``self_attn.out_proj.{weight,bias}``,
``self_attn_layer_norm.{weight,bias}``, ``fc1.{weight,bias}``, ``fc2.{weight,bias}``,
``final_layer_norm.{weight,bias}`` (reference:
metaseq/modules/transformer_decoder_layer.py:52-101; init options :103-177).

``forward`` picks between two implementations of the same math:
* the fused path (one autograd function over the sm_100a kernels,
  ``metaseq_b200.modules.fused_layer``) for 16-bit CUDA training / prefill without cache;
* the modular path (LayerNorm / attention / parallel linear modules) everywhere else:
  CPU, fp32, incremental decoding, dropout > 0, non-ReLU activations.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from metaseq_b200 import utils
from metaseq_b200.modules.activation_functions import ActivationFn
from metaseq_b200.modules.attention_bias import AttentionBias
from metaseq_b200.modules.dropout import Dropout
from metaseq_b200.modules.fused_layer import LayerSpec, fused_decoder_layer
from metaseq_b200.modules.layer_norm import LayerNorm
from metaseq_b200.modules.multihead_attention import ModelParallelMultiheadAttention
from metaseq_b200.ops import functional as ops_f
from metaseq_b200.parallel import mpu
from metaseq_b200.parallel.layers import ColumnParallelLinear, RowParallelLinear


# Tests set this to run the fused layer function on CPU / fp32 through the PyTorch
# restatements of the operators, which checks the hand-written backward exactly.
FORCE_FUSED_LAYER = False


def _get(args, name, default=None):
    return getattr(args, name, default)


class ModelParallelTransformerDecoderLayer(nn.Module):
    def __init__(self, args):
        super().__init__()
        self.args = args
        self.embed_dim = args.decoder_embed_dim
        self.sequence_parallel = bool(_get(args, "sequence_parallel", False))
        self.dropout_module = Dropout(_get(args, "dropout", 0.0), module_name=self.__class__.__name__)
        self.num_layers = args.decoder_layers
        dtype = utils.get_precise_dtype(args) if _get(args, "tensor_parallel_init_model_on_gpu", False) or \
            _get(args, "init_dtype_from_flags", False) else None
        device = torch.cuda.current_device() if (_get(args, "tensor_parallel_init_model_on_gpu", False)
                                                 and torch.cuda.is_available()) else None
        cpu_init = not _get(args, "tensor_parallel_init_model_on_gpu", False)
        full_init = bool(_get(args, "full_megatron_init", False))
        sigma = _get(args, "megatron_init_sigma", 0.006)
        scalar = _get(args, "full_megatron_init_scalar", 1.0)
        disable_bias = bool(_get(args, "disable_bias", False))
        affine = not bool(_get(args, "disable_affine_ln", False))
        ffn_dim = args.decoder_ffn_embed_dim
        self.activation_name = _get(args, "activation_fn", "relu") or "relu"

        self._build = dict(dtype=dtype, device=device, cpu_init=cpu_init)
        self.self_attn = self.build_self_attention(self.embed_dim, args)
        self.self_attn_layer_norm = LayerNorm(self.embed_dim, elementwise_affine=affine)
        truncate = bool(_get(args, "truncate_init", False))
        fc1 = self.build_fc1(self.embed_dim, ffn_dim, not cpu_init, full_init, sigma * scalar, dtype,
                             disable_bias=disable_bias, truncate_init=truncate)
        self.activation_fn = ActivationFn(self.activation_name, self._plain_fc1, self.embed_dim, ffn_dim,
                                          bias=not disable_bias, init=self.fc1_init_method, cpu_init=cpu_init,
                                          dtype=dtype, device=device, sp=self.sequence_parallel)
        self.fc1 = fc1  # registered after the activation's own parameters, which keeps the parameter order
        self.fc2 = self.build_fc2(ffn_dim, self.embed_dim, not cpu_init, full_init, scalar, sigma, self.num_layers,
                                  dtype, disable_bias=disable_bias, truncate_init=truncate)
        self.final_layer_norm = LayerNorm(self.embed_dim, elementwise_affine=affine)
        self.checkpoint_activations = bool(_get(args, "checkpoint_activations", False))
        self.offload_activations = bool(_get(args, "offload_activations", False))
        self.distribute_checkpointed_activations = bool(_get(args, "distribute_checkpointed_activations", False))
        self.use_fused_layer = not bool(_get(args, "no_fused_layer", False))
        self.tp_comm = None  # set by the trainer when fused tensor-parallel communication is on

    # ------------------------------------------------------------- builders (override points)
    def build_self_attention(self, embed_dim, args):
        b = self._build
        return ModelParallelMultiheadAttention(
            embed_dim, args.decoder_attention_heads, dropout=_get(args, "attention_dropout", 0.0),
            bias=not bool(_get(args, "disable_bias", False)), use_cpu_initialization=b["cpu_init"],
            full_megatron_init=bool(_get(args, "full_megatron_init", False)),
            full_megatron_init_scalar=_get(args, "full_megatron_init_scalar", 1.0),
            megatron_init_sigma=_get(args, "megatron_init_sigma", 0.006), num_layers=args.decoder_layers,
            dtype=b["dtype"], device=b["device"], sequence_parallel=self.sequence_parallel,
            max_positions=_get(args, "max_target_positions", None) or _get(args, "tokens_per_sample", 2048))

    @staticmethod
    def _default_weight_init(w):
        import math

        return nn.init.kaiming_uniform_(w, a=math.sqrt(5))

    def build_fc1(self, input_dim, output_dim, initialize_params_on_gpu, full_megatron_init, megatron_init_sigma,
                  dtype, disable_bias=False, truncate_init=False):
        """Column-parallel first feed-forward matrix.  ``megatron_init_sigma`` is the standard deviation actually
        used (the caller has multiplied in ``--full-megatron-init-scalar``)."""
        if full_megatron_init:
            self.fc1_init_method = utils.init_method_normal(megatron_init_sigma)
        else:
            self.fc1_init_method = self._default_weight_init
        return self._plain_fc1(input_dim, output_dim, bias=not disable_bias, init=self.fc1_init_method,
                               cpu_init=not initialize_params_on_gpu, dtype=dtype, device=self._build["device"],
                               sp=self.sequence_parallel)

    def build_fc2(self, input_dim, output_dim, initialize_params_on_gpu, full_megatron_init, full_megatron_init_scalar,
                  megatron_init_sigma, num_layers, dtype, disable_bias=False, truncate_init=False):
        """Row-parallel second feed-forward matrix (its input is already split over the tensor-parallel ranks)."""
        if full_megatron_init:
            init = utils.scaled_init_method_normal(megatron_init_sigma * full_megatron_init_scalar, num_layers)
        else:
            init = self._default_weight_init
        return RowParallelLinear(input_dim, output_dim, bias=not disable_bias, input_is_parallel=True,
                                 init_method=init, skip_bias_add=False,
                                 use_cpu_initialization=not initialize_params_on_gpu, dtype=dtype,
                                 device=self._build["device"], sequence_parallel=self.sequence_parallel)

    def forward_attention(self, query, key, value, residual, key_padding_mask=None, incremental_state=None,
                          attn_mask=None, bt=None):
        """Self-attention, its bias, dropout and the residual of the modular path (self-attention only: ``key`` and
        ``value`` are the query)."""
        if bt is None:
            bt = (query.shape[0], query.shape[1])
        h, attn_bias = self.self_attn(query, bt, incremental_state=incremental_state,
                                      key_padding_mask=key_padding_mask, attn_mask=attn_mask)
        if attn_bias is not None:
            h = h + attn_bias
        return residual + self.dropout_module(h).view_as(residual)

    @staticmethod
    def _plain_fc1(embed_dim, ffn_dim, bias, init, cpu_init, dtype, device, sp):
        return ColumnParallelLinear(embed_dim, ffn_dim, bias=bias, gather_output=False, init_method=init,
                                    use_cpu_initialization=cpu_init, dtype=dtype, device=device, sequence_parallel=sp)

    # Under FSDP with peer-memory collectives the four weight matrices may still be arriving from other
    # ranks when forward starts: the fused path reads them only through ``ops.functional.gemm``, which polls
    # the arrival flags per tile; every other path calls ``ensure_operand_ready`` first.
    supports_operand_flags = True
    operand_flag_parameters = ("self_attn.qkv_proj.weight", "self_attn.out_proj.weight", "fc1.weight", "fc2.weight")

    # ------------------------------------------------------------------ paths
    def _fused_ok(self, x, incremental_state, key_padding_mask, attn_mask) -> bool:
        if not self.use_fused_layer or incremental_state is not None or key_padding_mask is not None \
                or not (attn_mask is None or isinstance(attn_mask, AttentionBias)):
            return False  # dense masks take the modular path; document starts / ALiBi slopes go to the kernel
        if not (ops_f.use_kernels(x) or FORCE_FUSED_LAYER) or self.activation_name != "relu":
            return False
        if (not ops_f.attn_head_dim_ok(self.self_attn.head_dim) and not FORCE_FUSED_LAYER) or self.embed_dim % 8 != 0:
            return False
        if self.self_attn.qkv_proj.weight.dtype != x.dtype:
            return False
        return True

    def forward(self, x, bt: Optional[Tuple[int, int]] = None, incremental_state: Optional[Dict] = None,
                self_attn_padding_mask=None, self_attn_mask=None, recompute: Optional[bool] = None):
        """``x``: ``[B, T, D]`` (``[B*T/p, D]`` with sequence parallelism; then ``bt`` is required)."""
        if bt is None:
            bt = (x.shape[0], x.shape[1])
        if self._fused_ok(x, incremental_state, self_attn_padding_mask, self_attn_mask):
            a = self.self_attn
            if self.tp_comm is None and mpu.get_tensor_model_parallel_world_size() > 1 and x.is_cuda:
                from metaseq_b200.parallel import symm

                # every fused row-parallel product of the layer has a [B*T, D] result
                self.tp_comm = symm.get_tp_comm(mpu.get_tensor_model_parallel_group(), x.device, bt[0] * bt[1],
                                                self.embed_dim, x.dtype)
            seeds, p_res, p_attn = None, 0.0, 0.0
            if self.training and (self.dropout_module.p > 0 or self.self_attn.dropout_module.p > 0):
                # Three mask seeds per call from the host generator (reseeded per update by the trainer, so runs are
                # reproducible and no device sync is needed).  Residual masks are shared by the tensor-parallel
                # ranks (they hold the same activations) unless the sequence is sharded; attention heads differ
                # per rank, so that seed is offset by the rank.
                base = torch.randint(0, 2 ** 62, (3,), dtype=torch.int64).tolist()
                tp_rank = mpu.get_tensor_model_parallel_rank()
                res_off = tp_rank if self.sequence_parallel else 0
                seeds = (base[0] + 7919 * tp_rank, base[1] + res_off, base[2] + res_off)
                p_res, p_attn = float(self.dropout_module.p), float(self.self_attn.dropout_module.p)
            spec = LayerSpec(
                B=bt[0], T=bt[1], heads_local=a.num_heads_partition, head_dim=a.head_dim, scale=a.scaling,
                eps=self.self_attn_layer_norm.eps, tp_group=mpu.get_tensor_model_parallel_group(),
                tp_world=mpu.get_tensor_model_parallel_world_size(), sequence_parallel=self.sequence_parallel,
                recompute=self.checkpoint_activations if recompute is None else recompute, comm=self.tp_comm,
                dropout_p=p_res, attn_dropout_p=p_attn, seeds=seeds,
                doc_start=self_attn_mask.doc_start if self_attn_mask is not None else None,
                alibi_slopes=self_attn_mask.slopes if self_attn_mask is not None else None)
            ln1, ln2 = self.self_attn_layer_norm, self.final_layer_norm
            weights = (ln1.weight, ln1.bias, a.qkv_proj.weight, a.qkv_proj.bias, a.out_proj.weight, a.out_proj.bias,
                       ln2.weight, ln2.bias, self.fc1.weight, self.fc1.bias, self.fc2.weight, self.fc2.bias)
            park_input = spec.recompute and self.training and torch.is_grad_enabled() and \
                (self.offload_activations or self.distribute_checkpointed_activations)
            if park_input:
                # --offload-activations / --distribute-checkpointed-activations: the one tensor that recomputation
                # keeps (the layer input) goes to host memory or is split over the tensor-parallel ranks, and the
                # whole layer runs again in backward (with its own activations kept that second time)
                import dataclasses

                from .checkpoint_activations import checkpoint

                kept = dataclasses.replace(spec, recompute=False)
                return checkpoint(lambda t: fused_decoder_layer(t, kept, *weights), self, x,
                                  offload_to_cpu=self.offload_activations,
                                  distribute_checkpointed_activations=self.distribute_checkpointed_activations)
            return fused_decoder_layer(x, spec, *weights)
        # the library ops of the modular path do not poll arrival flags: wait for the matrices here
        for w in (self.self_attn.qkv_proj.weight, self.self_attn.out_proj.weight, self.fc1.weight, self.fc2.weight):
            ops_f.ensure_operand_ready(w)
        wanted = self.checkpoint_activations if recompute is None else recompute
        if wanted and self.training and incremental_state is None and torch.is_grad_enabled():
            # the modular path keeps only the layer input and recomputes the rest in backward, as the fused path
            # does inside its own backward
            from .checkpoint_activations import checkpoint

            return checkpoint(self._modular_forward, self, x, bt, None, self_attn_padding_mask, self_attn_mask,
                              offload_to_cpu=self.offload_activations,
                              distribute_checkpointed_activations=self.distribute_checkpointed_activations)
        return self._modular_forward(x, bt, incremental_state, self_attn_padding_mask, self_attn_mask)

    def _modular_forward(self, x, bt, incremental_state, key_padding_mask, attn_mask):
        h = self.self_attn_layer_norm(x)
        x = self.forward_attention(h, h, h, x, key_padding_mask=key_padding_mask,
                                   incremental_state=incremental_state, attn_mask=attn_mask, bt=bt)
        residual = x
        h = self.final_layer_norm(x)
        fc1_out, _ = self.fc1(h)
        h = self.activation_fn(h, fc1_out, model_parallel=True)
        h, _ = self.fc2(h)
        h = self.dropout_module(h)
        return residual + h.view_as(residual)

    def make_generation_fast_(self, **kwargs):
        pass
