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
from typing import Any, Dict, List, Optional

import torch

from metaseq_b200.checkpoint import flat_shards
from metaseq_b200.file_io import torch_load_cpu

from metaseq_b200.checkpoint._cli import add_option, add_switch  # noqa: E402

logger = logging.getLogger(__name__)


def _sorted_shards(pattern: str) -> List[str]:
    files = glob.glob(pattern)

    def key(p):
        m = re.search(r"shard(\d+)", os.path.basename(p))
        return int(m.group(1)) if m else 0

    return sorted(files, key=key)


_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def _cast(t, dtype: Optional[torch.dtype]):
    return t.to(dtype) if dtype is not None and torch.is_tensor(t) and t.is_floating_point() else t


def reshard_fsdp_model_weights(shard_weights: List[Dict[str, torch.Tensor]], shard_metadata: List[Dict[str, Any]],
                               num_output_shards: int = 1, unflatten_weights: bool = False,
                               dtype: Optional[torch.dtype] = None):
    """In memory: the ``model`` dicts and ``shard_metadata`` of every input shard -> ``(weights, metadata)``, one
    entry per output shard.  With ``unflatten_weights`` (one output shard only) the flat vectors are split back
    into named tensors (reference: metaseq/scripts/reshard_fsdp.py:143-206)."""
    if len(shard_weights) != len(shard_metadata):
        raise ValueError("Expect shard weights and shard metadata to have same length.")
    if unflatten_weights and num_output_shards > 1:
        raise ValueError("Unflatten weights only if the number of output shards is 1.")
    states = [{"model": w, "shard_metadata": m} for w, m in zip(shard_weights, shard_metadata)]
    if unflatten_weights:
        model = unflatten_state(states)["model"]
        return [{k: _cast(v, dtype) for k, v in model.items()}], [shard_metadata[0]]
    weights, metadata = [], []
    for r in range(num_output_shards):
        w, m = flat_shards.reshard_model_state(states, r, num_output_shards)
        weights.append({k: _cast(v, dtype) for k, v in w.items()})
        metadata.append(m)
    return weights, metadata


def reshard_fsdp_optim_state(shard_optim_states: List[Dict[str, Any]], shard_metadata: List[Dict[str, Any]],
                             shard_weights: List[Dict[str, torch.Tensor]], num_output_shards: int = 1,
                             dtype: Optional[torch.dtype] = None) -> List[Dict[str, Any]]:
    """In memory: every input shard's optimizer state -> one per output shard.  The i-th optimizer entry belongs
    to the i-th flat parameter, whose padding comes from the metadata (reference:
    metaseq/scripts/reshard_fsdp.py:209-250, which is handed the paddings as a list)."""
    if any("state" not in s for s in shard_optim_states):
        raise ValueError("Each sharded optimizer state dict should contain `state`.")
    states = [{"model": w, "shard_metadata": m, "last_optimizer_state": o}
              for w, m, o in zip(shard_weights, shard_metadata, shard_optim_states)]
    out = []
    for r in range(num_output_shards):
        st = flat_shards.reshard_optimizer_state(states, r, num_output_shards)
        st["state"] = {i: {k: _cast(v, dtype) if torch.is_tensor(v) and v.dim() > 0 else v for k, v in e.items()}
                       for i, e in st["state"].items()}
        out.append(st)
    return out


def reshard_fsdp_state_dicts(shard_state_dicts: List[Dict[str, Any]], num_output_shards: int = 1,
                             unflatten_weights: bool = True, skip_optimizer_state: bool = False,
                             dtype: Optional[torch.dtype] = None, drop_metaseq_req: bool = False) -> List[Dict[str, Any]]:
    """In memory: the checkpoint dicts of all shards of one model part -> ``num_output_shards`` checkpoint dicts.
    Everything but weights, metadata and optimizer state is copied from the first shard; ``drop_metaseq_req``
    removes the data iterator's state when it carries a tokenizer cache, which only unpickles with this package
    importable (reference: metaseq/scripts/reshard_fsdp.py:81-140)."""
    logger.info(f"Resharding state dicts into {num_output_shards} shard(s)")
    weights, metadata = reshard_fsdp_model_weights(
        [s["model"] for s in shard_state_dicts], [s.get("shard_metadata") for s in shard_state_dicts],
        num_output_shards, unflatten_weights, dtype)
    out: List[Dict[str, Any]] = []
    for w, m in zip(weights, metadata):
        out.append({"model": w} if unflatten_weights else {"model": w, "shard_metadata": m})
    if not skip_optimizer_state and not unflatten_weights and "last_optimizer_state" in shard_state_dicts[0]:
        opt = reshard_fsdp_optim_state(
            [s["last_optimizer_state"] for s in shard_state_dicts], [s.get("shard_metadata") for s in shard_state_dicts],
            [s["model"] for s in shard_state_dicts], num_output_shards, dtype)
        for d, o in zip(out, opt):
            d["last_optimizer_state"] = o
    first = shard_state_dicts[0]
    if drop_metaseq_req:
        itr = (first.get("extra_state") or {}).get("train_iterator")
        if isinstance(itr, dict) and "tokenization_cache" in itr:
            first = dict(first, extra_state=dict(first["extra_state"], train_iterator=None))
    for key, val in first.items():
        if key not in ("model", "shard_metadata", "last_optimizer_state"):
            for d in out:
                d[key] = val
    return out


def reshard_fsdp_checkpoints(src_dir_pattern: str, dst_dir_pattern: str, num_output_shards: int = 1,
                             unflatten_weights: bool = False, skip_optimizer_state: bool = False,
                             output_dtype: Optional[str] = None, drop_metaseq_req: bool = False) -> List[str]:
    if output_dtype and output_dtype not in _DTYPES:
        raise ValueError(f"The specified output dtype {output_dtype} is not supported.")
    paths = _sorted_shards(src_dir_pattern)
    if not paths:
        raise ValueError(f"The glob pattern {src_dir_pattern} doesn't match any sharded checkpoints.")
    logger.info(f"Loading {len(paths)} shards")
    states = [torch_load_cpu(p) for p in paths]
    new_states = reshard_fsdp_state_dicts(states, num_output_shards, unflatten_weights, skip_optimizer_state,
                                          _DTYPES.get(output_dtype), drop_metaseq_req)
    written = []
    for r, new in enumerate(new_states):
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
    add_option(ap, "--src-dir-pattern", "--input", dest="src_dir_pattern", required=True, help="glob of the input shards")
    add_option(ap, "--dst-dir-pattern", "--output", dest="dst_dir_pattern", required=True,
               help="output path with an {i} placeholder for the shard index")
    add_option(ap, "--num-output-shards", type=int, default=1)
    add_switch(ap, "--unflatten-weights", help="split flat parameters back into named tensors (one output shard)")
    add_switch(ap, "--skip-optimizer-state")
    add_option(ap, "--output-dtype", choices=sorted(_DTYPES), default=None, help="convert floating-point weights")
    add_switch(ap, "--drop-metaseq-req",
                    help="drop the data iterator state, which needs this package to unpickle")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    for p in reshard_fsdp_checkpoints(a.src_dir_pattern, a.dst_dir_pattern, a.num_output_shards, a.unflatten_weights,
                                      a.skip_optimizer_state, a.output_dtype, a.drop_metaseq_req):
        print(p)


if __name__ == "__main__":
    main()
