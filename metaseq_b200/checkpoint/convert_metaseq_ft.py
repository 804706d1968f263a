"""Exports consolidated, unflattened model-parallel checkpoints as FasterTransformer-style weight lists
(reference: metaseq/scripts/convert_metaseq_ft.py).

    python -m metaseq_b200.checkpoint.convert_metaseq_ft \
        --input "ckpt/reshard_no_os_unflat/reshard-model_part-*.pt" --output "ckpt-ft/part-{i}.pt" --dtype fp16

Per part the output is ``{"weights": [...]}``: for each of the twelve per-layer tensors below, the N layers in
order, then the final LayerNorm, the positional table without its two offset rows, and the token embedding
(concatenated over the parts) twice (input embedding and output projection).  Matrices are stored
input-major (transposed from ``nn.Linear``); the fused projection is reordered from this framework's
k, v, q row blocks to q, k, v and laid out ``[in, 3, out_per_part]``.  ``--quantize`` adds symmetric int8
weights with one scale per output column for the four large matrices of every layer."""
from __future__ import annotations

import argparse
import logging
import os
import re
from glob import glob
from typing import Any, Dict, List, Tuple

import torch

from metaseq_b200.checkpoint._cli import add_switch

logging.basicConfig(format="%(asctime)s | %(name)s | %(message)s", level=logging.INFO)
logger = logging.getLogger("metaseq_b200.checkpoint.convert_metaseq_ft")

_DTYPES = {"fp16": torch.float16, "fp32": torch.float32, "bf16": torch.bfloat16}


def _kvq_to_qkv(t: torch.Tensor) -> torch.Tensor:
    k, v, q = t.view(3, t.size(0) // 3, *t.shape[1:]).unbind(0)
    stacked = torch.stack([q, k, v], dim=0)
    return stacked if t.dim() == 1 else stacked.permute(2, 0, 1).contiguous()


def _transposed(t):
    return t.t().contiguous()


def _same(t):
    return t


# (key inside "decoder.layers.<i>.", transform), in the order the consumer expects
_PER_LAYER = [
    ("self_attn_layer_norm.weight", _same), ("self_attn_layer_norm.bias", _same),
    ("self_attn.qkv_proj.weight", _kvq_to_qkv), ("self_attn.qkv_proj.bias", lambda b: _kvq_to_qkv(b).view(3, -1)),
    ("self_attn.out_proj.weight", _transposed), ("self_attn.out_proj.bias", _same),
    ("final_layer_norm.weight", _same), ("final_layer_norm.bias", _same),
    ("fc1.weight", _transposed), ("fc1.bias", _same),
    ("fc2.weight", _transposed), ("fc2.bias", _same),
]
_QUANTIZED_SLOTS = (2, 4, 8, 10)  # qkv, out_proj, fc1, fc2 weights


def num_layers_of(state_dict: Dict[str, Any]) -> int:
    pat = re.compile(r"decoder\.layers\.(\d+)\.fc1\.weight")
    return 1 + max(int(m.group(1)) for m in map(pat.match, state_dict) if m)


def symmetric_int8_last_axis(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-column symmetric quantisation of ``[in, out]``: ``w ~ q * scale[out]``."""
    w32 = w.float()
    scale = w32.abs().amax(dim=0).clamp_min(1e-8) / 127.0
    q = torch.clamp(torch.round(w32 / scale), -127, 127).to(torch.int8)
    return q, scale.to(w.dtype)


def int8_weight_only_quantize(weights: List[torch.Tensor], num_layers: int) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
    """The four matrix slots of the consumer's weight list (fused projection, output projection, the two
    feed-forward matrices) as int8 with one scale per output column; their 16-bit copies are emptied in place.
    The reference calls the consumer library's own quantiser for this (metaseq/scripts/convert_metaseq_ft.py:99-133);
    the same symmetric per-column rule is computed here."""
    q_w: List[torch.Tensor] = []
    q_s: List[torch.Tensor] = []
    for slot in _QUANTIZED_SLOTS:
        for i in range(num_layers):
            w = weights[slot * num_layers + i]
            q, s = symmetric_int8_last_axis(w.flatten(1) if w.dim() == 3 else w)
            q_w.append(q)
            q_s.append(s)
            weights[slot * num_layers + i] = w.new_empty(0)
    return q_w, q_s


def convert_weights(state_dict, embedding_tokens, dtype, quantize=False) -> Dict[str, List[torch.Tensor]]:
    n = num_layers_of(state_dict)
    weights: List[torch.Tensor] = []
    for key, fn in _PER_LAYER:
        for i in range(n):
            weights.append(fn(state_dict[f"decoder.layers.{i}.{key}"].to(dtype)))
    weights.append(state_dict["decoder.layer_norm.weight"].to(dtype))
    weights.append(state_dict["decoder.layer_norm.bias"].to(dtype))
    weights.append(state_dict["decoder.embed_positions.weight"][2:])
    weights += [embedding_tokens, embedding_tokens]
    out = {"weights": weights}
    if quantize:
        out["int8_weights"], out["int8_scales"] = int8_weight_only_quantize(weights, n)
    return out


def convert_metaseq_ft(input: str, output: str, dtype: str = "fp16", quantize: bool = False) -> None:
    files = sorted(glob(input), key=lambda p: [int(x) for x in re.findall(r"\d+", p)])
    if not files:
        raise ValueError("The glob pattern doesn't match any model parallel parts.")
    logger.info(f"Found {len(files)} model parallel parts ({files[0]} to {files[-1]})")
    torch_dtype = _DTYPES[dtype]
    embed = torch.cat([torch.load(f, map_location="cpu", weights_only=False)["model"]["decoder.embed_tokens.weight"]
                       for f in files]).to(torch_dtype)
    for i, path in enumerate(files):
        logger.info(f"Converting {path}")
        sd = torch.load(path, map_location="cpu", weights_only=False)["model"]
        target = output.format(i=i)
        os.makedirs(os.path.dirname(os.path.abspath(target)), exist_ok=True)
        torch.save(convert_weights(sd, embed, torch_dtype, quantize), target)
        logger.info(f"Wrote {target}")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True, help="glob of the model-parallel parts")
    ap.add_argument("--output", required=True, help="output pattern; {i} is replaced by the part index")
    ap.add_argument("--dtype", default="fp16", choices=sorted(_DTYPES))
    add_switch(ap, "--quantize")
    a = ap.parse_args(argv)
    convert_metaseq_ft(a.input, a.output, a.dtype, a.quantize)


if __name__ == "__main__":
    main()
