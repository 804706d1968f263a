"""Quantisation noise ("Training with Quantization Noise for Extreme Model Compression"): during training,
random blocks of a layer's weight are zeroed (and the rest rescaled) in a forward pre-hook, so the model becomes
robust to later block-wise quantisation (reference: metaseq/modules/quant_noise.py).  Supported layers:
``nn.Linear``, ``nn.Embedding`` and ``nn.Conv2d``; ``p = 0`` leaves the module untouched."""
from __future__ import annotations

import torch
import torch.nn as nn


def _block_mask(module, weight: torch.Tensor, p: float, block_size: int) -> torch.Tensor:
    """Boolean mask shaped like ``weight``: True where the weight is dropped."""
    if isinstance(module, nn.Conv2d) and module.kernel_size != (1, 1):
        # whole kernels are dropped
        keep = torch.zeros(weight.size(0), weight.size(1), device=weight.device).bernoulli_(p)
        return keep.bool()[:, :, None, None].expand_as(weight)
    out_features = weight.size(0)
    in_features = weight[0].numel()
    drop = torch.zeros(in_features // block_size * out_features, device=weight.device).bernoulli_(p)
    return drop.view(out_features, -1).repeat_interleave(block_size, dim=-1).view_as(weight).bool()


def quant_noise(module, p: float, block_size: int):
    if p <= 0:
        return module
    assert isinstance(module, (nn.Linear, nn.Embedding, nn.Conv2d))
    if isinstance(module, nn.Conv2d) and module.kernel_size != (1, 1):
        k = module.kernel_size[0] * module.kernel_size[1]
        assert k % block_size == 0, "Kernel size must be a multiple of block size"
    elif isinstance(module, nn.Conv2d):
        assert module.in_channels % block_size == 0, "Input channels must be a multiple of block sizes"
    else:
        assert module.weight.size(1) % block_size == 0, "Input features must be a multiple of block sizes"

    def _noise(mod, _inputs):
        if not mod.training:
            return
        w = mod.weight
        mask = _block_mask(mod, w, p, block_size)
        mod.weight.data = w.masked_fill(mask, 0) / (1 - p)

    module.register_forward_pre_hook(_noise)
    return module
