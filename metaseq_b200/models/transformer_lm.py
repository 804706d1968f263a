"""``model_parallel_transformer_lm``: the OPT / GPT decoder-only language model and its
architectures (reference: metaseq/models/transformer_lm.py:32-339).

``build_model`` pads the dictionary to a multiple of 8 (times the tensor-parallel size),
builds the vocab-parallel embedding with either the ``N(0, D^-0.5)`` default or the
"full megatron" ``N(0, sigma)`` initialisation with a zero pad row, and checks the
sequence-parallel preconditions (tensor parallel > 1, dropout 0, ReLU/GELU).
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from metaseq_b200 import utils
from metaseq_b200.dataclass.configs import MetaseqDataclass, opt
from metaseq_b200.dataclass.constants import ATTN_CHOICES, UNSPECIFIED_DOC_SEP
from metaseq_b200.models import register_model, register_model_architecture
from metaseq_b200.models.base_model import LanguageModel
from metaseq_b200.models.transformer_decoder import ModelParallelTransformerDecoder
from metaseq_b200.parallel import mpu
from metaseq_b200.parallel.layers import VocabParallelEmbedding

logger = logging.getLogger(__name__)

DEFAULT_MAX_TARGET_POSITIONS = 1024
DEFAULT_MIN_PARAMS_TO_WRAP = int(1e8)


@dataclass
class TransformerLanguageModelConfig(MetaseqDataclass):
    activation_fn: str = opt("relu", "activation function to use", choices=utils.get_available_activation_fns())
    dropout: float = opt(0.1, "dropout probability")
    attention_dropout: float = opt(0.0, "dropout probability for attention weights")
    decoder_embed_dim: int = opt(512, "decoder embedding dimension")
    decoder_ffn_embed_dim: int = opt(2048, "decoder embedding dimension for FFN")
    decoder_layers: int = opt(6, "num decoder layers")
    decoder_attention_heads: int = opt(8, "num decoder attention heads")
    share_decoder_input_output_embed: bool = opt(False, "share decoder input and output embeddings")
    decoder_learned_pos: bool = opt(False, "use learned positional embeddings in the decoder")
    decoder_learned_sinusoidal: bool = opt(False, "use learned positional embeddings init with sinusoidal")
    no_scale_embedding: bool = opt(False, "if True, dont scale embeddings")
    checkpoint_activations: bool = opt(False, "checkpoint activations at each layer")
    offload_activations: bool = opt(False, "move checkpointed activations to CPU after they are used")
    min_params_to_wrap: int = opt(DEFAULT_MIN_PARAMS_TO_WRAP, "minimum number of params for a layer to be wrapped "
                                  "with FSDP() when training with --ddp-backend=fully_sharded")
    alibi: bool = opt(False, "use the ALiBi position method instead of regular position embeddings")
    self_attn_doc_sep: int = opt(UNSPECIFIED_DOC_SEP, "use dynamic self attention masking when document separator "
                                 "is specified")
    fsdp_checkpoint_wrap_layer_frequency: int = opt(1, "group transformer blocks and wrap the group in checkpoint "
                                                    "and FSDP wrapper together")
    distribute_checkpointed_activations: bool = opt(False, "distribute offloaded checkpoints to tensor parallel gpus")
    tensor_parallel_init_model_on_gpu: bool = opt(False, "initialize model directly on gpu and possibly fp16 for "
                                                  "tensor parallel")
    full_megatron_init: bool = opt(False, "exact same init as Megatron")
    full_megatron_init_scalar: float = opt(1.0, "factor to scale sigma by for the main layers in full megatron init")
    pos_init_scalar: float = opt(1.0, "factor to scale positional embedding init by")
    truncate_init: bool = opt(False, "truncate gaussian init to +/- 3 stddevs")
    megatron_init_sigma: float = opt(0.006, "sigma for megatron initialization")
    no_emb_dropout: Optional[bool] = opt(False, "avoid emb dropout for decoder")
    disable_bias: Optional[bool] = opt(False, "disable bias for all linear layers in transformer decoder")
    disable_affine_ln: Optional[bool] = opt(False, "disable weight and bias of layer norm")
    attn_variant: str = opt("default", "attention implementation hint", choices=("default",) + tuple(ATTN_CHOICES))
    xf_attn_op: str = opt("None", "kept for command-line compatibility; attention always uses the in-tree kernels")
    recompute_fc1_num_layers: Optional[int] = opt(0, "number of layers that recompute the fc1 output in backward")
    no_fused_layer: bool = opt(False, "run decoder layers through separate modules instead of the fused layer function")


@register_model("model_parallel_transformer_lm", dataclass=TransformerLanguageModelConfig)
class ModelParallelTransformerLanguageModel(LanguageModel):
    @classmethod
    def build_model(cls, args, task):
        base_lm_architecture(args)
        tp = mpu.get_tensor_model_parallel_world_size()
        task.source_dictionary.pad_to_multiple_(8 * tp)
        task.target_dictionary.pad_to_multiple_(8 * tp)
        if getattr(args, "sequence_parallel", False):
            assert getattr(args, "dropout", 0.0) == 0.0 and getattr(args, "attention_dropout", 0.0) == 0.0, \
                "sequence parallel requires dropout 0"
            assert args.activation_fn in ("relu", "gelu"), "sequence parallel supports relu / gelu"
        if getattr(args, "max_target_positions", None) is None:
            args.max_target_positions = getattr(args, "tokens_per_sample", DEFAULT_MAX_TARGET_POSITIONS)
        embed_tokens = cls.build_embedding(args, task.source_dictionary, args.decoder_embed_dim)
        decoder = ModelParallelTransformerDecoder(args, task.target_dictionary, embed_tokens)
        model = cls(decoder)
        dt = utils.get_precise_dtype(args)
        if dt != torch.float32 and getattr(args, "ddp_backend", None) == "fully_sharded":
            # sharded units are built from parameters that already have the training dtype
            model = model.to(dt)
        return model

    @classmethod
    def build_embedding(cls, args, dictionary, embed_dim, path=None):
        sigma = getattr(args, "megatron_init_sigma", 0.006)
        if getattr(args, "full_megatron_init", False):
            init = utils.init_method_normal(sigma)
        else:
            init = utils.init_method_normal(embed_dim ** -0.5)
        on_gpu = getattr(args, "tensor_parallel_init_model_on_gpu", False) and torch.cuda.is_available()
        dtype = utils.get_precise_dtype(args) if (on_gpu or getattr(args, "init_dtype_from_flags", False)) else None
        return VocabParallelEmbedding(
            len(dictionary), embed_dim, dictionary.pad(), init_method=init, use_cpu_initialization=not on_gpu,
            dtype=dtype, device=torch.cuda.current_device() if on_gpu else None)


@register_model("transformer_lm", dataclass=TransformerLanguageModelConfig)
class TransformerLanguageModel(ModelParallelTransformerLanguageModel):
    """The model under the name the reference keeps for a decoder without tensor parallelism
    (metaseq/models/transformer_lm.py:188-191, where it has no builder of its own).  With a tensor-parallel group
    of one the parallel layers are ordinary layers, so the same class serves both names."""


def base_lm_architecture(args):
    d = lambda k, v: setattr(args, k, getattr(args, k, v) if getattr(args, k, None) is not None else v)
    d("activation_fn", "relu")
    d("dropout", 0.1)
    d("attention_dropout", 0.0)
    d("decoder_embed_dim", 512)
    d("decoder_ffn_embed_dim", 2048)
    d("decoder_layers", 6)
    d("decoder_attention_heads", 8)
    d("share_decoder_input_output_embed", False)
    d("decoder_learned_pos", False)
    d("decoder_learned_sinusoidal", False)
    d("no_scale_embedding", False)
    d("add_bos_token", False)


@register_model_architecture("model_parallel_transformer_lm", "transformer_lm_megatron")
def transformer_lm_megatron(args):
    d = lambda k, v: setattr(args, k, getattr(args, k, v) if getattr(args, k, None) is not None else v)
    d("decoder_embed_dim", 3072)
    d("decoder_ffn_embed_dim", 3072 * 4)
    d("decoder_layers", 72)
    d("decoder_attention_heads", 32)
    d("dropout", 0.1)
    d("attention_dropout", 0.1)
    d("activation_fn", "gelu")
    base_lm_architecture(args)


@register_model_architecture("model_parallel_transformer_lm", "transformer_lm_gpt")
def transformer_lm_gpt(args):
    d = lambda k, v: setattr(args, k, getattr(args, k, v) if getattr(args, k, None) is not None else v)
    d("decoder_embed_dim", 768)
    d("decoder_ffn_embed_dim", 3072)
    d("decoder_layers", 12)
    d("decoder_attention_heads", 12)
    d("dropout", 0.1)
    d("attention_dropout", 0.1)
    d("activation_fn", "gelu")
    base_lm_architecture(args)


@register_model_architecture("model_parallel_transformer_lm", "transformer_lm_gpt2_tiny")
def transformer_lm_gpt2_tiny(args):
    d = lambda k, v: setattr(args, k, getattr(args, k, v) if getattr(args, k, None) is not None else v)
    d("decoder_embed_dim", 64)
    d("decoder_ffn_embed_dim", 64)
    d("decoder_layers", 2)
    d("decoder_attention_heads", 1)
    d("dropout", 0.1)
    d("attention_dropout", 0.1)
    d("activation_fn", "gelu")
    base_lm_architecture(args)


# Hyper-parameters of the published OPT family (embed dim, FFN = 4x, layers, heads), usable as
# ``--arch opt_<size>`` on top of the generic architectures above.
OPT_SIZES = {
    "125m": (768, 12, 12),
    "350m": (1024, 24, 16),
    "1.3b": (2048, 24, 32),
    "2.7b": (2560, 32, 32),
    "6.7b": (4096, 32, 32),
    "13b": (5120, 40, 40),
    "30b": (7168, 48, 56),
    "66b": (9216, 64, 72),
    "175b": (12288, 96, 96),
}


def apply_opt_defaults(args, size: str):
    dim, layers, heads = OPT_SIZES[size]
    d = lambda k, v: setattr(args, k, getattr(args, k, v) if getattr(args, k, None) is not None else v)
    d("decoder_embed_dim", dim)
    d("decoder_ffn_embed_dim", 4 * dim)
    d("decoder_layers", layers)
    d("decoder_attention_heads", heads)
    d("activation_fn", "relu")
    d("dropout", 0.1)
    d("attention_dropout", 0.1)
    args.share_decoder_input_output_embed = True
    args.decoder_learned_pos = True
    args.no_scale_embedding = True
    args.full_megatron_init = True
    d("megatron_init_sigma", 0.006)
    base_lm_architecture(args)


def _register_opt(size):
    name = "opt_" + size.replace(".", "_")

    @register_model_architecture("model_parallel_transformer_lm", name)
    def _arch(args, _size=size):
        apply_opt_defaults(args, _size)

    return _arch


for _s in OPT_SIZES:
    _register_opt(_s)
