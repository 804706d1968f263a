"""Parity with an independent implementation of the architecture: a random-initialised ``transformers``
``OPTForCausalLM`` and this framework's decoder, holding the same weights, give the same logits and the same
greedy continuation (the reference checks this against a downloaded OPT-125M:
gpu_tests/test_hf_compatibility.py:120-158; there is no network here, so both sides start from one random state)."""
import pytest
import torch

from metaseq_b200 import options, tasks
from metaseq_b200.dataclass.utils import convert_namespace_to_config

transformers = pytest.importorskip("transformers")

D, LAYERS, HEADS, FFN, MAXPOS = 64, 3, 4, 256, 48


def _ours():
    argv = ["--task", "dummy_lm", "--dict-size", "92", "--tokens-per-sample", str(MAXPOS), "--batch-size", "1",
            "--arch", "transformer_lm_megatron", "--decoder-layers", str(LAYERS), "--decoder-embed-dim", str(D),
            "--decoder-ffn-embed-dim", str(FFN), "--decoder-attention-heads", str(HEADS), "--decoder-learned-pos",
            "--share-decoder-input-output-embed", "--no-scale-embedding", "--activation-fn", "relu", "--dropout", "0.0",
            "--attention-dropout", "0.0", "--criterion", "cross_entropy", "--optimizer", "adam", "--lr", "1e-3", "--cpu",
            "--distributed-world-size", "1"]
    cfg = convert_namespace_to_config(options.parse_args_and_arch(options.get_training_parser(), input_args=argv))
    task = tasks.setup_task(cfg.task)
    torch.manual_seed(0)
    model = task.build_model(cfg.model).eval()
    with torch.no_grad():  # make every parameter non-trivial (biases and norms start at 0 / 1)
        for p in model.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    return model, task


def _hf_with_weights_of(model):
    from transformers import OPTConfig, OPTForCausalLM

    dec = model.decoder
    vocab = dec.embed_tokens.weight.shape[0]
    cfg = OPTConfig(vocab_size=vocab, hidden_size=D, num_hidden_layers=LAYERS, ffn_dim=FFN, num_attention_heads=HEADS,
                    max_position_embeddings=dec.embed_positions.weight.shape[0] - 2, do_layer_norm_before=True,
                    word_embed_proj_dim=D, activation_function="relu", dropout=0.0, attention_dropout=0.0,
                    pad_token_id=1, bos_token_id=0, eos_token_id=2, enable_bias=True, layer_norm_elementwise_affine=True)
    hf = OPTForCausalLM(cfg).eval()
    sd = {"model.decoder.embed_tokens.weight": dec.embed_tokens.weight,
          "model.decoder.embed_positions.weight": dec.embed_positions.weight,
          "model.decoder.final_layer_norm.weight": dec.layer_norm.weight,
          "model.decoder.final_layer_norm.bias": dec.layer_norm.bias,
          "lm_head.weight": dec.embed_tokens.weight}
    for i, layer in enumerate(dec.layers):
        pre = f"model.decoder.layers.{i}."
        a = layer.self_attn
        w, b = a.qkv_proj.weight, a.qkv_proj.bias  # rows packed as (k | v | q)
        for j, name in enumerate(("k_proj", "v_proj", "q_proj")):
            sd[pre + f"self_attn.{name}.weight"] = w[j * D:(j + 1) * D]
            sd[pre + f"self_attn.{name}.bias"] = b[j * D:(j + 1) * D]
        sd[pre + "self_attn.out_proj.weight"], sd[pre + "self_attn.out_proj.bias"] = a.out_proj.weight, a.out_proj.bias
        sd[pre + "self_attn_layer_norm.weight"] = layer.self_attn_layer_norm.weight
        sd[pre + "self_attn_layer_norm.bias"] = layer.self_attn_layer_norm.bias
        sd[pre + "fc1.weight"], sd[pre + "fc1.bias"] = layer.fc1.weight, layer.fc1.bias
        sd[pre + "fc2.weight"], sd[pre + "fc2.bias"] = layer.fc2.weight, layer.fc2.bias
        sd[pre + "final_layer_norm.weight"] = layer.final_layer_norm.weight
        sd[pre + "final_layer_norm.bias"] = layer.final_layer_norm.bias
    missing, unexpected = hf.load_state_dict({k: v.detach().clone() for k, v in sd.items()}, strict=False)
    assert not unexpected and all("lm_head" in m or "embed_tokens" in m for m in missing), (missing, unexpected)
    return hf


def test_logits_and_greedy_continuation_match_transformers_opt():
    model, task = _ours()
    hf = _hf_with_weights_of(model)
    tokens = torch.randint(4, 90, (3, 20), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        ours, _ = model(tokens)
        theirs = hf(input_ids=tokens).logits
    assert ours.shape == theirs.shape
    torch.testing.assert_close(ours, theirs, rtol=1e-4, atol=1e-4)
    # incremental decoding with the key/value cache against HF's generate (greedy)
    from metaseq_b200.sequence_generator import SequenceGenerator

    prompt = tokens[:, :8]
    sg = SequenceGenerator([model], task.target_dictionary, beam_size=1, max_len_b=16, min_len=16, temperature=1.0, topp=-1)
    mine = sg.generate([model], {"net_input": {"src_tokens": prompt}})["tokens"][:, 0, :15]
    with torch.no_grad():
        ref = hf.generate(prompt, max_new_tokens=7, do_sample=False, min_new_tokens=7,
                          suppress_tokens=[1, 2], pad_token_id=1)
    assert torch.equal(mine, ref[:, :15]), (mine, ref)
