"""Decoder stack: vocab-parallel token embedding + learned positions, N pre-LN layers,
final LayerNorm, tied output projection.

Behavioural contract from the reference (metaseq/models/transformer_decoder.py):
embedding = ``embed_scale * tok + pos`` with optional dropout (:263-346); under
sequence parallelism the activations are scattered across the tensor-parallel group
right after the embedding (:343-345); incremental decoding feeds only the new tokens
through the layers while positions are computed from the full prefix (:324-327);
logits stay vocabulary-sharded for the vocab-parallel criterion and are gathered
otherwise (:398-428); ``--self-attn-doc-sep`` restarts positions after every
separator token and blocks attention across documents (:270-313, :459-472).

Activations are batch-first ``[B, T, D]`` (sequence-parallel shards are
``[B*T/p, D]`` row blocks of the flattened tokens), so the final logits need no
transpose.
"""
from __future__ import annotations

import logging
import math
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from metaseq_b200 import utils
from metaseq_b200.dataclass.constants import UNSPECIFIED_DOC_SEP
from metaseq_b200.models.base_decoder import IncrementalDecoder
from metaseq_b200.modules.dropout import Dropout
from metaseq_b200.modules.layer_norm import LayerNorm
from metaseq_b200.modules.learned_positional_embedding import PositionalEmbedding
from metaseq_b200.modules.multihead_attention import KVCache
from metaseq_b200.modules.transformer_decoder_layer import ModelParallelTransformerDecoderLayer
from metaseq_b200.ops import autograd as ops_ag
from metaseq_b200.ops import functional as ops_f
from metaseq_b200.parallel import mappings, mpu


def _get(args, name, default=None):
    return getattr(args, name, default)



logger = logging.getLogger(__name__)


class TransformerDecoderMultiLayerBlockModule(nn.Module):
    """``--fsdp-checkpoint-wrap-layer-frequency N`` > 1: N consecutive decoder layers that are sharded as one unit
    (reference: metaseq/models/transformer_decoder.py:41-53, :123-157).  The call takes and returns what one layer
    takes and returns, so the decoder's loop does not change; activation recomputation stays inside each layer."""

    def __init__(self, layers):
        super().__init__()
        self.layers = nn.ModuleList(layers)

    def forward(self, x, **kwargs):
        for layer in self.layers:
            x = layer(x, **kwargs)
        return x


def log_weight_stats(tensor, name: str) -> None:
    """Mean, spread and range of a parameter at debug level (metaseq/models/transformer_decoder.py:56)."""
    if logger.isEnabledFor(logging.DEBUG):
        t = tensor.detach().float()
        logger.debug(f"{name}, mean: {t.mean():.5f}, std: {t.std():.5f}, min: {t.min():.5f}, max: {t.max():.5f}")


class _TiedProjection(nn.Module):
    """Holds the (shared) output-projection weight so that ``decoder.output_projection.weight``
    appears in the state dict next to ``decoder.embed_tokens.weight``."""

    def __init__(self, weight: nn.Parameter):
        super().__init__()
        self.weight = weight


class ModelParallelTransformerDecoder(IncrementalDecoder):
    def __init__(self, args, dictionary, embed_tokens):
        super().__init__(dictionary)
        self.args = args
        self.register_buffer("version", torch.Tensor([3]))
        self.padding_idx = embed_tokens.padding_idx
        self.embed_dim = args.decoder_embed_dim
        self.max_target_positions = _get(args, "max_target_positions", None) or _get(args, "tokens_per_sample", 2048)
        self.embed_tokens = embed_tokens
        log_weight_stats(embed_tokens.weight, "embed tokens")
        self.embed_scale = 1.0 if _get(args, "no_scale_embedding", False) else math.sqrt(self.embed_dim)
        self.sequence_parallel = bool(_get(args, "sequence_parallel", False))
        self.self_attn_doc_sep = _get(args, "self_attn_doc_sep", UNSPECIFIED_DOC_SEP)
        self.dropout_module = None
        if not _get(args, "no_emb_dropout", False) and _get(args, "dropout", 0.0) > 0:
            self.dropout_module = Dropout(args.dropout, module_name=self.__class__.__name__)
        dtype = embed_tokens.weight.dtype
        device = embed_tokens.weight.device if embed_tokens.weight.is_cuda else None
        self.embed_positions = None
        if _get(args, "decoder_learned_pos", False) and not _get(args, "alibi", False):
            self.embed_positions = PositionalEmbedding(
                self.max_target_positions, self.embed_dim, self.padding_idx, learned=True,
                learned_sinusoidal=_get(args, "decoder_learned_sinusoidal", False),
                full_megatron_init=_get(args, "full_megatron_init", False),
                pos_init_scalar=_get(args, "pos_init_scalar", 1.0),
                megatron_init_sigma=_get(args, "megatron_init_sigma", 0.006),
                truncate_init=_get(args, "truncate_init", False), dtype=dtype, device=device)
        group = int(_get(args, "fsdp_checkpoint_wrap_layer_frequency", 1) or 1)
        if group > 1:
            # several consecutive layers form one sharded unit (fewer, larger all-gathers and reduce-scatters);
            # parameter names become layers.<block>.layers.<i>.*
            assert args.decoder_layers % group == 0, "num layers should be divisible by checkpoint wrap frequency"
            from metaseq_b200.parallel.fsdp import fsdp_wrap

            raw = [self.build_decoder_layer(args, wrap=False) for _ in range(args.decoder_layers)]
            min_params = 0 if _get(args, "checkpoint_activations", False) else _get(args, "min_params_to_wrap", None)
            self.layers = nn.ModuleList([
                fsdp_wrap(TransformerDecoderMultiLayerBlockModule(raw[i:i + group]), min_num_params=min_params)
                for i in range(0, len(raw), group)])
        else:
            self.layers = nn.ModuleList([self.build_decoder_layer(args) for _ in range(args.decoder_layers)])
        if logger.isEnabledFor(logging.DEBUG):
            for name, param in self.layers.named_parameters():
                log_weight_stats(param, name)
        self.num_layers = args.decoder_layers
        self.layer_norm = LayerNorm(self.embed_dim, elementwise_affine=not _get(args, "disable_affine_ln", False))
        if dtype != torch.float32:
            self.layer_norm.to(dtype)
        if device is not None:
            self.layer_norm.to(device)
        if _get(args, "share_decoder_input_output_embed", False):
            self.output_projection = _TiedProjection(self.embed_tokens.weight)
        else:
            w = nn.Parameter(torch.empty_like(self.embed_tokens.weight))
            nn.init.normal_(w, mean=0, std=self.embed_dim ** -0.5)
            self.output_projection = _TiedProjection(w)
        self.inference = False
        self._cache_key = "decoder_state_" + str(id(self))
        # ALiBi: learned positions are off (above) and every head adds slope * key position to its scores; this
        # rank's heads are a contiguous slice of the slope list
        self.alibi_slopes = None
        if _get(args, "alibi", False):
            from metaseq_b200.modules.attention_bias import alibi_slopes

            tp, rank = mpu.get_tensor_model_parallel_world_size(), mpu.get_tensor_model_parallel_rank()
            per = args.decoder_attention_heads // tp
            self.alibi_slopes = torch.tensor(alibi_slopes(args.decoder_attention_heads)[rank * per:(rank + 1) * per],
                                             dtype=torch.float32)

    def build_decoder_layer(self, args, wrap: bool = True):
        layer = ModelParallelTransformerDecoderLayer(args)
        dt = utils.get_precise_dtype(args)
        if _get(args, "fp16", False) or _get(args, "memory_efficient_fp16", False) or _get(args, "bf16", False):
            layer = layer.to(dt)
        if not wrap:
            return layer
        from metaseq_b200.parallel.fsdp import fsdp_wrap

        return fsdp_wrap(layer, min_num_params=_get(args, "min_params_to_wrap", None))

    def buffered_future_mask(self, tensor, input_tokens=None):
        """The dense additive attention mask that the compact form stands for, for code that wants the matrix:
        ``[T, T]`` causal; ``[B, T, T]`` when documents are separated (``input_tokens`` required);
        ``[B * heads, T, T]`` with ALiBi.  ``tensor`` is ``[T, B, ...]`` and gives length, batch, dtype and
        device (reference: metaseq/models/transformer_decoder.py:436-487).  The model itself never builds it."""
        from metaseq_b200.modules.attention_bias import AttentionBias

        T, B = tensor.size(0), tensor.size(1)
        doc_start = None
        if self.self_attn_doc_sep != UNSPECIFIED_DOC_SEP:
            assert input_tokens is not None
            _, doc_start = self._doc_sep_positions(input_tokens)
        mask = AttentionBias(doc_start=doc_start, slopes=self.alibi_slopes).dense(T, T, 0, tensor.device)
        if self.alibi_slopes is not None:
            return mask.expand(B, -1, T, T).reshape(-1, T, T).to(tensor.dtype)
        if doc_start is not None:
            return mask[:, 0].to(tensor.dtype)
        return mask[0, 0].to(tensor.dtype)

    # ------------------------------------------------------------- embedding
    def _doc_sep_positions(self, tokens):
        """Positions that restart at ``padding_idx + 1`` after every separator token."""
        sep = tokens.eq(self.self_attn_doc_sep)
        starts = torch.zeros_like(tokens, dtype=torch.bool)
        starts[:, 1:] = sep[:, :-1]
        starts[:, 0] = True
        idx = torch.arange(tokens.shape[1], device=tokens.device).expand_as(tokens)
        last_start = torch.where(starts, idx, torch.zeros_like(idx)).cummax(dim=1)[0]
        mask = tokens.ne(self.padding_idx)
        return ((idx - last_start + 1) * mask).long() + self.padding_idx, last_start

    def forward_embedding(self, tokens, incremental_state=None, past: int = 0):
        doc_start = None
        if self.self_attn_doc_sep != UNSPECIFIED_DOC_SEP:
            positions, doc_start = self._doc_sep_positions(tokens)
        elif self.embed_positions is not None:
            positions = utils.make_positions(tokens, self.padding_idx)
        else:
            positions = None
        if past > 0:
            tokens = tokens[:, past:]
            if positions is not None:
                positions = positions[:, past:]
        w = self.embed_tokens.weight
        tp = mpu.get_tensor_model_parallel_world_size()
        pos_w = self.embed_positions.weight if (self.embed_positions is not None and positions is not None
                                                and hasattr(self.embed_positions, "weight")) else None
        if ops_f.use_kernels(w) and w.shape[1] % 8 == 0 and (pos_w is None or pos_w.dtype == w.dtype):
            if tp == 1:
                x = ops_ag.embedding(tokens, positions, w, pos_w, self.embed_scale, self.padding_idx, 0)
            else:
                x = ops_ag.embedding(tokens, None, w, None, self.embed_scale, self.padding_idx,
                                     self.embed_tokens.vocab_start_index)
                x = mappings.reduce_from_tensor_model_parallel_region(x)
                if pos_w is not None:
                    x = x + torch.nn.functional.embedding(positions, pos_w)
            embed = x
        else:
            embed = self.embed_scale * self.embed_tokens(tokens)
            x = embed
            if positions is not None and self.embed_positions is not None:
                if pos_w is not None:
                    x = x + torch.nn.functional.embedding(positions, pos_w, self.padding_idx)
                else:
                    x = x + self.embed_positions(tokens, positions=positions)
        if self.dropout_module is not None:
            x = self.dropout_module(x)
        return x, embed, positions, doc_start

    def _embedding_norm_sums(self, tokens, positions, x) -> dict:
        """Sums over tokens of the L2 norms of the token embedding, the position embedding and their sum (what the
        reference reads off ``inner_states[0]``, metaseq/criterions/vocab_parallel_cross_entropy.py:51-70).  The
        token part comes from the row norms of the table, so the fused embedding kernel needs no second output."""
        l2 = lambda t: torch.linalg.vector_norm(t.detach(), dim=-1, dtype=torch.float32)  # noqa: E731
        out = {"emb": l2(x).sum()}
        w = self.embed_tokens.weight
        row_norm = l2(w) * self.embed_scale
        tp = mpu.get_tensor_model_parallel_world_size()
        if tp == 1:
            out["tok"] = row_norm[tokens.reshape(-1)].sum()
        else:  # rows of other ranks count zero here; the sum over the tensor-parallel group completes it
            lo = self.embed_tokens.vocab_start_index
            local = tokens.reshape(-1) - lo
            mine = (local >= 0) & (local < w.shape[0])
            part = (row_norm[local.clamp(0, w.shape[0] - 1)] * mine).sum()
            torch.distributed.all_reduce(part, group=mpu.get_tensor_model_parallel_group())
            out["tok"] = part
        pos_w = getattr(self.embed_positions, "weight", None) if self.embed_positions is not None else None
        if pos_w is not None and positions is not None:
            out["pos"] = l2(pos_w)[positions.reshape(-1)].sum()
        return out

    # ---------------------------------------------------------------- forward
    def forward(self, prev_output_tokens, src_lengths=None, incremental_state=None, features_only: bool = False,
                self_attn_padding_mask=None, **unused):
        x, extra = self.extract_features(prev_output_tokens, incremental_state=incremental_state,
                                         self_attn_padding_mask=self_attn_padding_mask)
        if not features_only:
            x = self.output_layer(x, bt=extra["bt"], norm_sums=extra.get("norm_sums"))
        return x, extra

    def _past_length(self, incremental_state) -> int:
        if not incremental_state:
            return 0
        for v in incremental_state.values():
            if isinstance(v, KVCache):
                return v.length
        return 0

    def extract_features(self, prev_output_tokens, incremental_state=None, self_attn_padding_mask=None, **unused):
        past = self._past_length(incremental_state)
        B = prev_output_tokens.shape[0]
        x, tok_emb, positions, doc_start = self.forward_embedding(prev_output_tokens, incremental_state, past)
        T = x.shape[1]
        norms = None
        if self.training and incremental_state is None and _get(self.args, "log_activation_norms", True):
            with torch.no_grad():
                norms = self._embedding_norm_sums(prev_output_tokens, positions, x)
        # What attention sees beyond causality travels in its compact form: one document start per token (a token
        # attends only inside its own document; not applied while decoding incrementally) and one ALiBi slope per
        # head.  The flash-attention kernels take both directly; other paths expand them to an additive mask.
        attn_mask = None
        use_doc = doc_start is not None and incremental_state is None
        if use_doc or self.alibi_slopes is not None:
            from metaseq_b200.modules.attention_bias import AttentionBias

            if self.alibi_slopes is not None and self.alibi_slopes.device != x.device:
                self.alibi_slopes = self.alibi_slopes.to(x.device)
            attn_mask = AttentionBias(doc_start=doc_start.to(torch.int32) if use_doc else None,
                                      slopes=self.alibi_slopes)
        if self.sequence_parallel:
            x = mappings.scatter_to_sequence_parallel_region(x.reshape(B * T, -1))
        inner_states: List[Optional[torch.Tensor]] = []
        # --recompute-fc1-num-layers N: the first N layers give up their stored activations and recompute them in
        # backward, whether or not --checkpoint-activations asks that of every layer (the reference recomputes only
        # the first feed-forward product of those layers; the fused layer here recomputes as a whole)
        early = int(_get(self.args, "recompute_fc1_num_layers", 0) or 0)
        per_block = max(1, self.num_layers // max(1, len(self.layers)))
        for idx, layer in enumerate(self.layers):
            extra = {"recompute": True} if idx * per_block < early and self.training else {}
            x = layer(x, bt=(B, T), incremental_state=incremental_state,
                      self_attn_padding_mask=self_attn_padding_mask, self_attn_mask=attn_mask, **extra)
        x = self.layer_norm(x)
        return x, {"inner_states": inner_states, "tok_emb": tok_emb, "positions": positions, "bt": (B, T),
                   "norm_sums": norms}

    def output_layer(self, features, **kwargs):
        """Project to the vocabulary with the (tied) embedding matrix."""
        w = self.output_projection.weight
        tp = mpu.get_tensor_model_parallel_world_size()
        if self.sequence_parallel:
            features = mappings.gather_from_sequence_parallel_region(features, True)
        elif tp > 1:
            features = mappings.copy_to_tensor_model_parallel_region(features)
        if kwargs.get("norm_sums") is not None:  # final activations, all positions (after the sequence gather)
            with torch.no_grad():
                kwargs["norm_sums"]["actv"] = torch.linalg.vector_norm(features.detach(), dim=-1, dtype=torch.float32).sum()
        vocab_parallel = _get(self.args, "criterion", None) == "vocab_parallel_cross_entropy"
        gather = tp > 1 and (self.inference or not vocab_parallel)
        # Training straight into a cross entropy: the product also leaves the softmax pieces of every row, where
        # that pays: under tensor parallelism (it replaces a pass over the logits and a library collective) and for
        # vocabularies whose rows do not fit the one-pass kernel's shared memory.  On one rank with a row that fits,
        # that kernel reads and writes the logits once, and the statistics epilogue would only slow the product
        # (measured at 16384 x 50272: 2.84 instead of 2.54 ms).
        want_stats = self.training and not gather and torch.is_grad_enabled() and \
            (tp > 1 or w.shape[0] * w.element_size() > 200 * 1024)
        if ops_f.use_kernels(features) and features.dtype == w.dtype and w.shape[0] % 8 == 0:
            logits = ops_ag.linear(features, w, row_stats=want_stats)
        else:
            logits = torch.nn.functional.linear(features, w)
        row_stats = getattr(logits, "_msq_row_stats", None)
        if gather:
            logits = mappings.gather_from_tensor_model_parallel_region(logits)
        if logits.dim() == 2 and "bt" in kwargs:
            logits = logits.view(*kwargs["bt"], -1)
        if row_stats is not None:
            logits._msq_row_stats = row_stats
        return logits

    def max_positions(self):
        if self.embed_positions is None:
            return self.max_target_positions
        return min(self.max_target_positions, self.embed_positions.max_positions)

    def make_generation_fast_(self, **kwargs):
        self.inference = True

    def upgrade_state_dict_named(self, state_dict, name):
        key = f"{name}.version" if name else "version"
        if key not in state_dict:
            state_dict[key] = torch.Tensor([3])
        return state_dict
