"""Change the tensor-parallel size of a consolidated (unflattened) checkpoint.

    python -m metaseq_b200.checkpoint.reshard_mp --src-dir-pattern "reshard-model_part-*.pt" \
        --dst-dir-pattern "out/reshard-model_part-{i}.pt" --num-output-parts 4

Keys are classified by name (reference: metaseq/scripts/reshard_mp.py:17-119 and
metaseq/distributed/stitch_fsdp_ckpt.py:246-351): split along dim 0 (embeddings, fc1, q/k/v
projections), split along dim 1 (fc2 / out_proj weights), replicated (positions, layer norms,
fc2 / out_proj biases, version).  The fused ``qkv_proj`` is viewed as ``[3, rows/3, ...]`` so
that the k | v | q blocks of every input part are merged block-wise and re-chunked block-wise.
"""
from __future__ import annotations

import argparse
import glob
import logging
import os
import re
from typing import Any, Dict, List

import torch

from metaseq_b200.file_io import torch_load_cpu

from metaseq_b200.checkpoint._cli import add_option, add_switch  # noqa: E402

logger = logging.getLogger(__name__)

DIM0 = re.compile(r"embed_tokens|output_projection|ffn_layernorm|fc1|(k|q|v)_proj")
DIM1 = re.compile(r"(fc2|out_proj)\.weight")
SHARED = re.compile(r"embed_positions|layer_norm|(fc2|out_proj)\.bias|version")


def _sorted_parts(pattern: str) -> List[str]:
    files = glob.glob(pattern)

    def key(p):
        m = re.search(r"model_part-(\d+)", os.path.basename(p))
        return int(m.group(1)) if m else 0

    return sorted(files, key=key)


def merge_parts(tensors: List[torch.Tensor], key: str) -> torch.Tensor:
    if "qkv_proj" in key:
        viewed = [t.view(3, t.shape[0] // 3, *t.shape[1:]) for t in tensors]
        merged = torch.cat(viewed, dim=1)
        return merged.reshape(-1, *tensors[0].shape[1:])
    if SHARED.search(key):
        for t in tensors[1:]:
            if t.shape != tensors[0].shape or not torch.allclose(t.float(), tensors[0].float(), atol=1e-3, rtol=1e-3):
                logger.warning(f"replicated tensor {key} differs between parts; keeping part 0")
                break
        return tensors[0]
    if DIM1.search(key):
        return torch.cat(tensors, dim=1)
    if DIM0.search(key):
        return torch.cat(tensors, dim=0)
    return tensors[0]


def split_part(t: torch.Tensor, key: str, n: int) -> List[torch.Tensor]:
    if "qkv_proj" in key:
        v = t.view(3, t.shape[0] // 3, *t.shape[1:])
        return [c.reshape(-1, *t.shape[1:]).clone() for c in v.chunk(n, dim=1)]
    if SHARED.search(key):
        return [t.clone() for _ in range(n)]
    if DIM1.search(key):
        return [c.clone() for c in t.chunk(n, dim=1)]
    if DIM0.search(key):
        return [c.clone() for c in t.chunk(n, dim=0)]
    return [t.clone() for _ in range(n)]


def reshard_megatron_parts(model_parts, new_model_part_count: int = 1) -> List[Dict[str, torch.Tensor]]:
    """In-memory form: ``model_parts`` (a list, or a dict keyed by part index, of unflattened state dicts of one
    model) re-cut into ``new_model_part_count`` parts; one part is the whole model
    (metaseq/distributed/stitch_fsdp_ckpt.py:246-351)."""
    if isinstance(model_parts, dict):
        model_parts = [model_parts[k] for k in sorted(model_parts)]
    out: List[Dict[str, torch.Tensor]] = [dict() for _ in range(new_model_part_count)]
    for key in model_parts[0]:
        tensors = [part[key] for part in model_parts]
        if not torch.is_tensor(tensors[0]):
            for o in out:
                o[key] = tensors[0]
            continue
        whole = merge_parts(tensors, key) if len(tensors) > 1 else tensors[0]
        for o, piece in zip(out, split_part(whole, key, new_model_part_count)):
            o[key] = piece
    return out


def get_n_layers(glued_model: Dict[str, Any]) -> int:
    """Number of decoder layers in a state dict, counted from its ``decoder.layers.<i>.fc1.weight`` keys."""
    n = 0
    while f"decoder.layers.{n}.fc1.weight" in glued_model:
        n += 1
    assert n > 0, "found 0 layers: no key decoder.layers.0.fc1.weight"
    return n


def find_num_parts(names) -> int:
    """Number of tensor-parallel parts among file names (largest ``-model_part-<i>`` + 1; 0 when none has one)."""
    found = [int(m.group(1)) for m in (re.search(r"-model_part-(\d+)", n) for n in names) if m is not None]
    return max(found) + 1 if found else 0


def reshard_mp(src_dir_pattern: str, dst_dir_pattern: str, num_output_parts: int = 1, drop_optimizer_state: bool = True):
    paths = _sorted_parts(src_dir_pattern)
    assert len(paths) > 0, f"no files match {src_dir_pattern}"
    states = [torch_load_cpu(p) for p in paths]
    keys = list(states[0]["model"].keys())
    merged = {k: merge_parts([s["model"][k] for s in states], k) for k in keys}
    outs = [dict() for _ in range(num_output_parts)]
    for k, t in merged.items():
        for i, piece in enumerate(split_part(t, k, num_output_parts)):
            outs[i][k] = piece
    written = []
    for i, model in enumerate(outs):
        st = {k: v for k, v in states[0].items() if k != "model"}
        if drop_optimizer_state:
            st.pop("last_optimizer_state", None)
        st.pop("shard_metadata", None)
        st["model"] = model
        cfg = st.get("cfg")
        if isinstance(cfg, dict):
            if isinstance(cfg.get("common"), dict):
                cfg["common"]["model_parallel_size"] = num_output_parts
            m = cfg.get("model")
            if m is not None:
                if isinstance(m, dict):
                    m["model_parallel_size"] = num_output_parts
                else:
                    setattr(m, "model_parallel_size", num_output_parts)
        dst = dst_dir_pattern.format(i=i)
        os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
        torch.save(st, dst)
        written.append(dst)
    return written


def reshard_model_parallel_parts(input: str, output: str, num_output_parts: int = 1, eps: float = 1e-8) -> List[str]:
    """The reference's entry point name and argument names (metaseq/scripts/reshard_mp.py:17-119): ``input`` is a
    glob over the parts, ``output`` a pattern with ``{i}``; tensors that every part replicates are taken from
    part 0, with a warning when another part's copy is further than ``eps`` away."""
    paths = _sorted_parts(input)
    if not paths:
        raise ValueError("The glob pattern doesn't match any model parallel parts.")
    first = torch_load_cpu(paths[0])["model"]
    for p in paths[1:]:
        other = torch_load_cpu(p)["model"]
        for key, t in first.items():
            if torch.is_tensor(t) and SHARED.search(key) and "qkv_proj" not in key and t.shape == other[key].shape:
                diff = float((t.float() - other[key].float()).abs().max()) if t.numel() else 0.0
                if diff > eps:
                    logger.warning(f"Max value discrepancy for key '{key}': {diff:.4e}")
    return reshard_mp(input, output, num_output_parts, drop_optimizer_state=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_option(ap, "--src-dir-pattern", "--input", dest="src_dir_pattern", required=True)
    add_option(ap, "--dst-dir-pattern", "--output", dest="dst_dir_pattern", required=True)
    add_option(ap, "--num-output-parts", type=int, default=1)
    add_switch(ap, "--keep-optimizer-state")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    for p in reshard_mp(a.src_dir_pattern, a.dst_dir_pattern, a.num_output_parts, not a.keep_optimizer_state):
        print(p)


if __name__ == "__main__":
    main()
