"""Merge all tensor-parallel parts of a consolidated checkpoint into a single-GPU state dict
(``restored.pt``), the format single-process tools consume (reference:
metaseq/scripts/convert_to_singleton.py, which gathers over NCCL; here the parts are merged on
the host from the files)."""
from __future__ import annotations

import argparse
import logging
import os

import torch

from metaseq_b200.checkpoint.reshard_mp import _sorted_parts, merge_parts
from metaseq_b200.file_io import torch_load_cpu

logger = logging.getLogger(__name__)


def convert_to_singleton(src_dir: str, prefix: str = "reshard", out_name: str = "restored.pt"):
    paths = _sorted_parts(os.path.join(src_dir, f"{prefix}-model_part-*.pt"))
    assert paths, f"no {prefix}-model_part-*.pt under {src_dir}"
    states = [torch_load_cpu(p) for p in paths]
    keys = list(states[0]["model"].keys())
    model = {k: merge_parts([s["model"][k] for s in states], k) for k in keys}
    out = {k: v for k, v in states[0].items() if k not in ("model", "last_optimizer_state", "shard_metadata")}
    out["model"] = model
    cfg = out.get("cfg")
    if isinstance(cfg, dict) and isinstance(cfg.get("common"), dict):
        cfg["common"]["model_parallel_size"] = 1
    dst = os.path.join(src_dir, out_name)
    torch.save(out, dst)
    return dst


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("location")
    ap.add_argument("--prefix", default="reshard")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    print(convert_to_singleton(a.location, a.prefix))


if __name__ == "__main__":
    main()
