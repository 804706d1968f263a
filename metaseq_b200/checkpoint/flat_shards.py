"""Arithmetic on flat-parameter shards: unpad, concatenate, re-slice, unflatten.

A sharded checkpoint stores, per FSDP unit, this rank's equal-sized slice of the unit's
flattened parameters; padding sits at the end of the last shard(s) and its amount per shard is
recorded in ``shard_metadata`` (reference consumers: metaseq/scripts/reshard_fsdp.py:158-265,
metaseq/checkpoint_utils.py:709-906).  Everything here works on the *logical* vector (all
shards concatenated with padding removed), so any old world size can be mapped to any new one,
and the same code serves parameters and per-parameter optimizer state.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch


def flat_keys(model_state: Dict[str, Any]) -> List[str]:
    return [k for k in model_state if k.endswith("flat_param_0")]


def metadata_by_key(shard_metadata: Dict[str, Any]) -> Dict[str, Dict[str, Any]]:
    """``{"<fsdp_path>.flat_param_0": {"names", "shapes", "numels", "padding"}}``."""
    out = {}
    for entry in (shard_metadata or {}).get("param_metadata", []):
        path = entry.get("fsdp_path", "")
        for flat_name, md in entry["params"].items():
            key = f"{path}.{flat_name}" if path else flat_name
            out[key] = md
    return out


def unpadded_numel(md: Dict[str, Any]) -> int:
    return int(sum(md["numels"]))


def shard_size_for(total: int, world: int) -> int:
    """Per-rank shard length used by this framework: equal shards, multiple of 8 elements."""
    n = (total + world - 1) // world
    return (n + 7) // 8 * 8


def logical_vector(shards: Sequence[torch.Tensor], paddings: Optional[Sequence[int]], total: Optional[int]) -> torch.Tensor:
    """Concatenates shards (in rank order) and strips padding.  Either per-shard paddings or the
    logical length must be known."""
    parts = []
    for i, s in enumerate(shards):
        s = s.reshape(-1)
        pad = int(paddings[i]) if paddings is not None else 0
        parts.append(s[: s.numel() - pad] if pad > 0 else s)
    vec = torch.cat(parts) if len(parts) > 1 else parts[0]
    if total is not None and vec.numel() > total:
        vec = vec[:total]
    return vec


def slice_for_rank(vec: torch.Tensor, rank: int, world: int, shard_numel: Optional[int] = None) -> Tuple[torch.Tensor, int]:
    """This rank's shard of the logical vector (zero padded) and the amount of padding in it."""
    total = vec.numel()
    n = shard_numel if shard_numel is not None else shard_size_for(total, world)
    start, end = rank * n, (rank + 1) * n
    out = vec.new_zeros(n)
    if start < total:
        take = min(end, total) - start
        out[:take] = vec[start:start + take]
    pad = min(n, max(0, end - total))
    return out, pad


def unflatten(vec: torch.Tensor, md: Dict[str, Any], prefix: str) -> Dict[str, torch.Tensor]:
    out = {}
    off = 0
    for name, shape, n in zip(md["names"], md["shapes"], md["numels"]):
        key = f"{prefix}.{name}" if prefix else name
        out[key] = vec[off:off + n].view(torch.Size(shape)).clone()
        off += n
    return out


def flatten(named: Dict[str, torch.Tensor], md: Dict[str, Any], prefix: str) -> torch.Tensor:
    parts = []
    for name, shape, n in zip(md["names"], md["shapes"], md["numels"]):
        key = f"{prefix}.{name}" if prefix else name
        t = named[key]
        assert t.numel() == n, f"{key}: {t.numel()} != {n}"
        parts.append(t.reshape(-1))
    return torch.cat(parts)


def reshard_model_state(states: Sequence[Dict[str, Any]], new_rank: int, new_world: int) -> Tuple[Dict[str, Any], Dict[str, Any]]:
    """``states``: the full checkpoint dicts of *all* old data-parallel shards of one model part,
    in rank order.  Returns ``(model_state, shard_metadata)`` for ``new_rank`` of ``new_world``."""
    mds = [metadata_by_key(s.get("shard_metadata")) for s in states]
    model0 = states[0]["model"]
    new_model: Dict[str, Any] = {}
    new_md_entries = []
    for key in model0:
        if not key.endswith("flat_param_0"):
            new_model[key] = model0[key]
            continue
        md = mds[0][key]
        total = unpadded_numel(md)
        vec = logical_vector([s["model"][key] for s in states], [m[key].get("padding", 0) for m in mds], total)
        shard, pad = slice_for_rank(vec, new_rank, new_world)
        new_model[key] = shard
        path = key[: -len("flat_param_0")].rstrip(".")
        new_md_entries.append({
            "fsdp_path": path,
            "params": {"flat_param_0": {"names": list(md["names"]), "shapes": list(md["shapes"]),
                                        "numels": list(md["numels"]), "padding": pad}},
            "no_broadcast_optim_state": False,
            "shared_param_info": [],
        })
    meta0 = states[0].get("shard_metadata") or {}
    # keep shared-parameter info from the source metadata
    src_entries = {e.get("fsdp_path", ""): e for e in meta0.get("param_metadata", [])}
    for e in new_md_entries:
        e["shared_param_info"] = list(src_entries.get(e["fsdp_path"], {}).get("shared_param_info", []))
    new_meta = {"param_metadata": new_md_entries, "buffer_names": list(meta0.get("buffer_names", []))}
    return new_model, new_meta


def reshard_optimizer_state(states: Sequence[Dict[str, Any]], new_rank: int, new_world: int) -> Optional[Dict[str, Any]]:
    """Re-slices per-parameter optimizer tensors (exp_avg, exp_avg_sq, ...) the same way.  The
    i-th optimizer parameter corresponds to the i-th flat parameter in state-dict order."""
    opt0 = states[0].get("last_optimizer_state")
    if not isinstance(opt0, dict) or "state" not in opt0:
        return opt0
    mds = [metadata_by_key(s.get("shard_metadata")) for s in states]
    keys = flat_keys(states[0]["model"])
    new_state = {}
    for idx, st in opt0["state"].items():
        key = keys[int(idx)] if int(idx) < len(keys) else None
        entry = {}
        for name, val in st.items():
            if torch.is_tensor(val) and val.dim() > 0 and key is not None and val.numel() == states[0]["model"][key].numel():
                total = unpadded_numel(mds[0][key])
                pieces = [s["last_optimizer_state"]["state"][idx] for s in states]
                if name + "_scale" in st:
                    # moments stored as scaled fp16: every shard has its own scale, so they are joined as fp32 and
                    # the optimizer compresses them again after its next step
                    tensors = [pc[name].float() * float(pc[name + "_scale"]) for pc in pieces]
                else:
                    tensors = [pc[name] for pc in pieces]
                vec = logical_vector(tensors, [m[key].get("padding", 0) for m in mds], total)
                entry[name], _ = slice_for_rank(vec, new_rank, new_world)
            elif name.endswith("_scale") and name[: -len("_scale")] in st:
                continue  # folded into the tensor above
            else:
                entry[name] = val
        new_state[idx] = entry
    out = {k: v for k, v in opt0.items() if k != "state"}
    out["state"] = new_state
    return out
