"""The hand-written backward of the fused decoder layer, checked on CPU in fp32 against
autograd through the modular layer (both use the PyTorch restatements of the operators)."""
import argparse

import pytest
import torch

from metaseq_b200.modules import transformer_decoder_layer as tdl


def _args(**kw):
    base = dict(decoder_embed_dim=32, decoder_attention_heads=4, decoder_ffn_embed_dim=64, decoder_layers=2,
                dropout=0.0, attention_dropout=0.0, activation_fn="relu", full_megatron_init=True,
                megatron_init_sigma=0.1, tokens_per_sample=16)
    base.update(kw)
    return argparse.Namespace(**base)


@pytest.mark.parametrize("recompute", [False, True])
@pytest.mark.parametrize("variant", ["default", "no_bias_no_affine"])
def test_fused_layer_backward_matches_autograd(recompute, variant):
    torch.manual_seed(0)
    kw = {}
    if variant == "no_bias_no_affine":
        kw = dict(disable_bias=True, disable_affine_ln=True)
    layer = tdl.ModelParallelTransformerDecoderLayer(_args(checkpoint_activations=recompute, **kw)).double()
    for n, p in layer.named_parameters():
        if n.endswith("bias") or "layer_norm" in n:
            torch.nn.init.normal_(p, std=0.2)
    x = torch.randn(2, 16, 32, dtype=torch.double, requires_grad=True)
    dy = torch.randn(2, 16, 32, dtype=torch.double)

    def run(fused):
        tdl.FORCE_FUSED_LAYER = fused
        try:
            for p in layer.parameters():
                p.grad = None
            x.grad = None
            assert layer._fused_ok(x, None, None, None) == fused
            y = layer(x)
            y.backward(dy)
            return y.detach().clone(), x.grad.clone(), {n: p.grad.clone() for n, p in layer.named_parameters()}
        finally:
            tdl.FORCE_FUSED_LAYER = False

    y1, dx1, g1 = run(True)
    y0, dx0, g0 = run(False)
    torch.testing.assert_close(y1, y0, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(dx1, dx0, rtol=1e-4, atol=1e-6)
    assert set(g1) == set(g0)
    for n in g0:
        torch.testing.assert_close(g1[n], g0[n], rtol=1e-4, atol=1e-6, msg=n)
