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


@pytest.mark.parametrize("which", ["documents", "alibi", "both"])
def test_document_starts_and_alibi_reach_the_fused_layer_and_match_the_dense_mask(which):
    """The compact form (one document start per token, one slope per head) through the fused layer equals the
    modular layer fed the additive ``[B, H, T, T]`` mask built the reference's way."""
    import math

    from metaseq_b200.modules.attention_bias import AttentionBias, alibi_slopes

    torch.manual_seed(1)
    B, T, D, H = 2, 16, 32, 4
    layer = tdl.ModelParallelTransformerDecoderLayer(_args()).double()
    x = torch.randn(B, T, D, dtype=torch.double, requires_grad=True)
    dy = torch.randn(B, T, D, dtype=torch.double)
    doc_start = torch.tensor([[0, 0, 0, 3, 3, 3, 3, 7, 7, 9, 9, 9, 9, 9, 14, 14], [0] * 5 + [5] * 11]) \
        if which in ("documents", "both") else None
    slopes = torch.tensor(alibi_slopes(H)) if which in ("alibi", "both") else None
    assert alibi_slopes(8)[0] == pytest.approx(0.5) and alibi_slopes(8)[-1] == pytest.approx(2.0 ** -8)
    assert len(alibi_slopes(12)) == 12 and alibi_slopes(12)[:8] == alibi_slopes(8)
    bias = AttentionBias(doc_start=doc_start, slopes=slopes)
    # the reference's construction: causal -inf above the diagonal, -inf across documents, slope * key position
    pos = torch.arange(T)
    dense = torch.zeros(B, H, T, T, dtype=torch.double)
    dense.masked_fill_((pos[None, :] > pos[:, None])[None, None], -math.inf)
    if doc_start is not None:
        dense.masked_fill_((pos.view(1, 1, T) < doc_start.view(B, T, 1))[:, None], -math.inf)
    if slopes is not None:
        dense = dense + slopes.double().view(1, H, 1, 1) * pos.double().view(1, 1, 1, T)
    torch.testing.assert_close(bias.dense(T, T, 0, x.device).double().expand(B, H, T, T), dense)

    def run(fused, mask):
        tdl.FORCE_FUSED_LAYER = fused
        try:
            for p in layer.parameters():
                p.grad = None
            x.grad = None
            assert layer._fused_ok(x, None, None, mask) == fused
            layer(x, self_attn_mask=mask).backward(dy)
            return x.grad.clone(), {n: p.grad.clone() for n, p in layer.named_parameters()}
        finally:
            tdl.FORCE_FUSED_LAYER = False

    dx1, g1 = run(True, bias)
    dx0, g0 = run(False, dense)
    dx_plain, _ = run(False, None)
    torch.testing.assert_close(dx1, dx0, rtol=1e-4, atol=1e-6)
    for n in g0:
        torch.testing.assert_close(g1[n], g0[n], rtol=1e-4, atol=1e-6, msg=n)
    assert not torch.allclose(dx1, dx_plain, atol=1e-4)  # the masks change the result


@pytest.mark.parametrize("dropout", [0.0, 0.2])
def test_offloaded_layer_input_gives_the_gradients_of_plain_recomputation(dropout):
    """``--offload-activations`` on the fused path: the layer input is parked outside and the layer runs again in
    backward; outputs and gradients equal those of the layer's own recomputation, dropout masks included."""
    def grads(offload):
        torch.manual_seed(0)
        layer = tdl.ModelParallelTransformerDecoderLayer(
            _args(checkpoint_activations=True, offload_activations=offload, dropout=dropout)).double()
        layer.train()
        x = torch.randn(2, 16, 32, dtype=torch.double, requires_grad=True)
        tdl.FORCE_FUSED_LAYER = True
        try:
            torch.manual_seed(7)  # the mask seeds are drawn from the host generator
            y = layer(x)
            y.square().sum().backward()
        finally:
            tdl.FORCE_FUSED_LAYER = False
        return y.detach(), x.grad, {n: p.grad for n, p in layer.named_parameters()}

    y0, dx0, g0 = grads(False)
    y1, dx1, g1 = grads(True)
    torch.testing.assert_close(y1, y0)
    torch.testing.assert_close(dx1, dx0)
    for n in g0:
        torch.testing.assert_close(g1[n], g0[n], msg=n)
