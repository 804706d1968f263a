"""Consolidate every model part of a sharded checkpoint into ``<prefix>-model_part-K.pt`` files
with unflattened weights and no optimizer state (inference format), optionally merging the
tensor-parallel parts into one file (reference: metaseq/scripts/consolidate_fsdp_shards.py and
metaseq/distributed/stitch_fsdp_ckpt.py)."""
from __future__ import annotations

import argparse
import glob
import logging
import os
import re
from typing import List

import torch

from metaseq_b200.checkpoint.reshard_fsdp import _sorted_shards, unflatten_state
from metaseq_b200.checkpoint.reshard_mp import merge_parts
from metaseq_b200.file_io import torch_load_cpu

from metaseq_b200.checkpoint._cli import add_option, add_switch  # noqa: E402

logger = logging.getLogger(__name__)


def find_model_parts(prefix: str) -> List[int]:
    parts = set()
    for f in glob.glob(prefix + "-model_part-*-shard*.pt"):
        m = re.search(r"model_part-(\d+)-shard", f)
        if m:
            parts.add(int(m.group(1)))
    return sorted(parts)


def consolidate_fsdp_shards(pth_prefix: str, save_prefix=None, new_arch_name=None, merge_model_parts: bool = False):
    """``pth_prefix``: path up to (not including) ``-model_part-K-shardN.pt``."""
    if pth_prefix.endswith(".pt"):
        pth_prefix = pth_prefix[:-3]
    save_prefix = save_prefix or pth_prefix + "_consolidated"
    parts = find_model_parts(pth_prefix)
    assert parts, f"no shards found for {pth_prefix}"
    consolidated = []
    for k in parts:
        paths = _sorted_shards(f"{pth_prefix}-model_part-{k}-shard*.pt")
        states = [torch_load_cpu(p) for p in paths]
        for s in states:
            s.pop("last_optimizer_state", None)
        out = unflatten_state(states)
        if new_arch_name is not None and isinstance(out.get("cfg"), dict) and out["cfg"].get("model") is not None:
            m = out["cfg"]["model"]
            if isinstance(m, dict):
                m["arch"] = m["_name"] = new_arch_name
            else:
                m.arch = m._name = new_arch_name
        consolidated.append(out)
    written = []
    if merge_model_parts and len(consolidated) > 1:
        keys = list(consolidated[0]["model"].keys())
        merged = dict(consolidated[0])
        merged["model"] = {key: merge_parts([c["model"][key] for c in consolidated], key) for key in keys}
        dst = f"{save_prefix}.pt"
        torch.save(merged, dst)
        written.append(dst)
    else:
        for k, out in zip(parts, consolidated):
            dst = f"{save_prefix}-model_part-{k}.pt"
            os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
            torch.save(out, dst)
            written.append(dst)
    return written


def consolidate_model_parallel(metadata, names, strict, weights, parts: int = 2, no_stitch_megatron: bool = False):
    """In memory: ``weights[i]`` / ``metadata[i]`` are the ``model`` dict and ``shard_metadata`` of the file called
    ``names[i]`` (``...part-<p>...``).  Every model part's shards are unflattened; the parts are then joined into one
    model unless ``no_stitch_megatron``, in which case ``{part: state dict}`` is returned (reference:
    metaseq/distributed/stitch_fsdp_ckpt.py:180-200; ``strict`` is accepted for the signature: a missing name
    always raises here)."""
    from metaseq_b200.checkpoint.reshard_mp import reshard_megatron_parts

    per_part = {}
    for p in range(parts):
        picked = [i for i, n in enumerate(names) if f"part-{p}" in n]
        if picked:
            states = [{"model": weights[i], "shard_metadata": metadata[i]} for i in picked]
            per_part[p] = unflatten_state(states)["model"]
    if no_stitch_megatron:
        return per_part
    return reshard_megatron_parts(per_part, new_model_part_count=1)[0]


def handle_qkv_proj(model_parts, key: str, new_model_part_count: int):
    """The fused projection of every part is three stacked blocks (K, V, Q order); each block is joined over the
    parts and cut again into ``new_model_part_count`` pieces.  Returns the three tuples of pieces (reference:
    metaseq/distributed/stitch_fsdp_ckpt.py:203-214)."""
    blocks = [model_parts[i][key].view(3, -1, *model_parts[i][key].shape[1:]) for i in range(len(model_parts))]
    joined = torch.cat(blocks, dim=1)
    return tuple(torch.chunk(joined[j], new_model_part_count) for j in range(3))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("pth_prefix")
    add_option(ap, "--save-prefix", default=None)
    add_option(ap, "--new-arch-name", default=None)
    add_switch(ap, "--merge-model-parts")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    for p in consolidate_fsdp_shards(a.pth_prefix, a.save_prefix, a.new_arch_name, a.merge_model_parts):
        print(p)


if __name__ == "__main__":
    main()
