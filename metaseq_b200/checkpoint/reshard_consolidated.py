"""Turn a consolidated (unflattened) checkpoint back into flat FSDP shards.

    python -m metaseq_b200.checkpoint.reshard_consolidated --src ckpt-model_part-0.pt \
        --dst-dir-pattern "out-model_part-0-shard{i}.pt" --num-output-shards 4

Parameters are grouped into units the way the trainer wraps them (one unit per decoder layer
plus a root unit), flattened in registration order, padded and chunked; ``shard_metadata`` is
regenerated so the result loads with ``--use-sharded-state`` (reference:
metaseq/scripts/reshard_consolidated.py:21-84).
"""
from __future__ import annotations

import argparse
import copy
import logging
import os
import re
from collections import OrderedDict
from typing import Any, Dict, List

import torch

from metaseq_b200.checkpoint import flat_shards
from metaseq_b200.file_io import torch_load_cpu

from metaseq_b200.checkpoint._cli import add_option, add_switch  # noqa: E402

logger = logging.getLogger(__name__)

LAYER_ORDER = [
    "self_attn.qkv_proj.weight", "self_attn.qkv_proj.bias", "self_attn.out_proj.weight", "self_attn.out_proj.bias",
    "self_attn_layer_norm.weight", "self_attn_layer_norm.bias", "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias",
    "final_layer_norm.weight", "final_layer_norm.bias",
]
ROOT_ORDER = ["decoder.embed_tokens.weight", "decoder.embed_positions.weight", "decoder.layer_norm.weight",
              "decoder.layer_norm.bias"]


def group_units(model: Dict[str, torch.Tensor]):
    units: "OrderedDict[str, List[str]]" = OrderedDict()
    units[""] = [k for k in ROOT_ORDER if k in model]
    layer_re = re.compile(r"^(decoder\.layers\.\d+)\.(.+)$")
    layers: Dict[str, List[str]] = OrderedDict()
    for k in model:
        m = layer_re.match(k)
        if m:
            layers.setdefault(m.group(1), []).append(m.group(2))
    for path, names in sorted(layers.items(), key=lambda kv: int(kv[0].rsplit(".", 1)[1])):
        ordered = [n for n in LAYER_ORDER if n in names] + [n for n in names if n not in LAYER_ORDER]
        units[path] = ordered
    return units


def reshard_consolidated(src: str, dst_dir_pattern: str, num_output_shards: int):
    state = torch_load_cpu(src)
    model = state["model"]
    units = group_units(model)
    buffers = {k: v for k, v in model.items() if k.endswith("version")}
    shared = []
    if "decoder.output_projection.weight" in model and "decoder.embed_tokens.weight" in model:
        shared = [("decoder.output_projection.weight", "decoder.embed_tokens.weight")]
    written = []
    for r in range(num_output_shards):
        new_model: Dict[str, Any] = dict(buffers)
        entries = []
        for path, names in units.items():
            if not names:
                continue
            full_names = [n if path == "" else f"{path}.{n}" for n in names]
            local_names = names if path != "" else names
            md = {"names": list(local_names), "shapes": [model[f].shape for f in full_names],
                  "numels": [model[f].numel() for f in full_names]}
            vec = torch.cat([model[f].reshape(-1) for f in full_names])
            shard, pad = flat_shards.slice_for_rank(vec, r, num_output_shards)
            key = f"{path}.flat_param_0" if path else "flat_param_0"
            new_model[key] = shard
            entries.append({"fsdp_path": path, "params": {"flat_param_0": dict(md, padding=pad)},
                            "no_broadcast_optim_state": False,
                            "shared_param_info": shared if path == "" else []})
        st = {k: v for k, v in state.items() if k not in ("model", "last_optimizer_state")}
        st["model"] = new_model
        st["shard_metadata"] = {"param_metadata": entries, "buffer_names": list(buffers.keys())}
        dst = dst_dir_pattern.format(i=r)
        os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
        torch.save(st, dst)
        written.append(dst)
    return written


def reshard_unflattened_model_weights(unsharded_weights: Dict[str, torch.Tensor], shard_metadata: Dict[str, Any],
                                      num_output_shards: int = 1):
    """In memory: named tensors plus the ``shard_metadata`` that says which names form which flat parameter ->
    ``(weights, metadata)`` with one flat, padded shard dict per output rank.  Buffers are copied to every shard.
    Used when the checkpoint already carries metadata (``reshard_consolidated`` derives the grouping from the
    parameter names instead).  Reference: metaseq/scripts/reshard_consolidated.py:53-84."""
    weights: List[Dict[str, torch.Tensor]] = [dict() for _ in range(num_output_shards)]
    for name in shard_metadata.get("buffer_names", []):
        if name not in unsharded_weights:
            raise ValueError(f"No buffer found for buffer name {name}.")
        for w in weights:
            w[name] = unsharded_weights[name]
    metadata = [copy.deepcopy(shard_metadata) for _ in range(num_output_shards)]
    for idx, entry in enumerate(shard_metadata["param_metadata"]):
        path = entry.get("fsdp_path", "")
        for flat_name, md in entry["params"].items():
            full = [f"{path}.{n}" if path else n for n in md["names"]]
            vec = torch.cat([unsharded_weights[f].reshape(-1) for f in full])
            key = f"{path}.{flat_name}" if path else flat_name
            for r in range(num_output_shards):
                weights[r][key], pad = flat_shards.slice_for_rank(vec, r, num_output_shards)
                metadata[r]["param_metadata"][idx]["params"][flat_name]["padding"] = pad
    return weights, metadata


def reshard_consolidated_checkpoint(input: str, output: str, num_output_shards: int = 1) -> List[str]:
    """The reference's entry point name and argument names (metaseq/scripts/reshard_consolidated.py:21-50).  A
    checkpoint that carries ``shard_metadata`` is cut along it; one without is grouped by parameter name."""
    state = torch_load_cpu(input)
    if not state.get("shard_metadata"):
        return reshard_consolidated(input, output, num_output_shards)
    weights, metadata = reshard_unflattened_model_weights(dict(state["model"]), state["shard_metadata"], num_output_shards)
    written = []
    for r in range(num_output_shards):
        st = {k: v for k, v in state.items() if k not in ("model", "shard_metadata", "optimizer_state",
                                                           "last_optimizer_state")}
        st["model"], st["shard_metadata"] = weights[r], metadata[r]
        dst = output.format(i=r)
        os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
        torch.save(st, dst)
        written.append(dst)
    return written


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_option(ap, "--src", "--input", dest="src", required=True)
    add_option(ap, "--dst-dir-pattern", "--output", dest="dst_dir_pattern", required=True)
    add_option(ap, "--num-output-shards", type=int, default=1)
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    for p in reshard_consolidated(a.src, a.dst_dir_pattern, a.num_output_shards):
        print(p)


if __name__ == "__main__":
    main()
