from .adaptive_softmax import AdaptiveSoftmax  # noqa: F401,E402
from .group_norm_fp32 import GroupNormFp32  # noqa: F401,E402
from .quant_noise import quant_noise  # noqa: F401,E402


# Names that the reference exports at package level, resolved on first use (importing them eagerly here would pull
# the kernel loader and the parallel layers into every ``import metaseq_b200.modules``).
_LAZY = {
    "ActivationFn": (".activation_functions", "ActivationFn"),
    "gelu": (".activation_functions", "gelu"),
    "Dropout": (".dropout", "Dropout"),
    "FeedForward": (".feedforward", "FeedForward"),
    "LayerNorm": (".layer_norm", "LayerNorm"),
    "LayerNormFp32": (".layer_norm", "LayerNormFp32"),
    "LearnedPositionalEmbedding": (".learned_positional_embedding", "LearnedPositionalEmbedding"),
    "PositionalEmbedding": (".learned_positional_embedding", "PositionalEmbedding"),
    "SinusoidalPositionalEmbedding": (".sinusoidal_positional_embedding", "SinusoidalPositionalEmbedding"),
    "Linear": (".linear", "Linear"),
    "ModelParallelMultiheadAttention": (".multihead_attention", "ModelParallelMultiheadAttention"),
    "ModelParallelTransformerDecoderLayer": (".transformer_decoder_layer", "ModelParallelTransformerDecoderLayer"),
    "FusedDecoderLayerFn": (".fused_layer", "FusedDecoderLayerFn"),
}


def __getattr__(name):
    try:
        module, attr = _LAZY[name]
    except KeyError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
    import importlib

    value = getattr(importlib.import_module(module, __name__), attr)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
