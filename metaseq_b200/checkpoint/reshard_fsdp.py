"""Reshard or consolidate the data-parallel (FSDP) shards of a checkpoint.

    python -m metaseq_b200.checkpoint.reshard_fsdp --src-dir-pattern "ckpt-model_part-0-shard*.pt" \
        --dst-dir-pattern "out-model_part-0-shard{i}.pt" --num-output-shards 2 [--unflatten-weights] \
        [--skip-optimizer-state]

Loads every input shard of one model part, strips each flat parameter's padding (from
``shard_metadata``), concatenates, and either re-chunks into ``num_output_shards`` equal shards
with fresh padding or (``--unflatten-weights``, single output shard) splits the flat vector back
into named tensors.  Optimizer state is resharded the same way.  Reference:
metaseq/scripts/reshard_fsdp.py:28-265.
"""
from __future__ import annotations

import argparse
import glob
import logging
import os
import re
from typing import Any, Dict, List

import torch

from metaseq_b200.checkpoint import flat_shards
from metaseq_b200.file_io import torch_load_cpu

logger = logging.getLogger(__name__)


def _sorted_shards(pattern: str) -> List[str]:
    files = glob.glob(pattern)

    def key(p):
        m = re.search(r"shard(\d+)", os.path.basename(p))
        return int(m.group(1)) if m else 0

    return sorted(files, key=key)


def reshard_fsdp_checkpoints(src_dir_pattern: str, dst_dir_pattern: str, num_output_shards: int = 1,
                             unflatten_weights: bool = False, skip_optimizer_state: bool = False) -> List[str]:
    paths = _sorted_shards(src_dir_pattern)
    assert len(paths) > 0, f"no files match {src_dir_pattern}"
    logger.info(f"Loading {len(paths)} shards")
    states = [torch_load_cpu(p) for p in paths]
    if skip_optimizer_state:
        for s in states:
            s.pop("last_optimizer_state", None)
    written = []
    if unflatten_weights:
        assert num_output_shards == 1, "unflattening produces a single consolidated file per model part"
        out = unflatten_state(states)
        dst = dst_dir_pattern.format(i=0)
        os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
        torch.save(out, dst)
        return [dst]
    for r in range(num_output_shards):
        new = {k: v for k, v in states[0].items() if k not in ("model", "shard_metadata", "last_optimizer_state")}
        new["model"], new["shard_metadata"] = flat_shards.reshard_model_state(states, r, num_output_shards)
        if not skip_optimizer_state and "last_optimizer_state" in states[0]:
            new["last_optimizer_state"] = flat_shards.reshard_optimizer_state(states, r, num_output_shards)
        dst = dst_dir_pattern.format(i=r)
        os.makedirs(os.path.dirname(os.path.abspath(dst)), exist_ok=True)
        torch.save(new, dst)
        written.append(dst)
    return written


def unflatten_state(states: List[Dict[str, Any]]) -> Dict[str, Any]:
    """One state dict with the original parameter names from all shards of a model part."""
    mds = [flat_shards.metadata_by_key(s.get("shard_metadata")) for s in states]
    model = {}
    for key, val in states[0]["model"].items():
        if not key.endswith("flat_param_0"):
            model[key] = val
            continue
        md = mds[0][key]
        vec = flat_shards.logical_vector([s["model"][key] for s in states], [m[key].get("padding", 0) for m in mds],
                                         flat_shards.unpadded_numel(md))
        prefix = key[: -len("flat_param_0")].rstrip(".")
        model.update(flat_shards.unflatten(vec, md, prefix))
    meta = states[0].get("shard_metadata") or {}
    for entry in meta.get("param_metadata", []):
        path = entry.get("fsdp_path", "")
        for shared, src in entry.get("shared_param_info", []):
            a = f"{path}.{shared}" if path else shared
            b = f"{path}.{src}" if path else src
            if b in model:
                model[a] = model[b]
    out = {k: v for k, v in states[0].items() if k not in ("model", "shard_metadata", "last_optimizer_state")}
    out["model"] = model
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--src-dir-pattern", required=True)
    ap.add_argument("--dst-dir-pattern", required=True, help="output path with an {i} placeholder for the shard index")
    ap.add_argument("--num-output-shards", type=int, default=1)
    ap.add_argument("--unflatten-weights", action="store_true")
    ap.add_argument("--skip-optimizer-state", action="store_true")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    for p in reshard_fsdp_checkpoints(a.src_dir_pattern, a.dst_dir_pattern, a.num_output_shards, a.unflatten_weights,
                                      a.skip_optimizer_state):
        print(p)


if __name__ == "__main__":
    main()
