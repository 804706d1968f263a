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


def create_generation_config_with_defaults(model_path: str, ddp_backend: str = "pytorch_ddp"):
    """A generation config for the checkpoint directory ``model_path`` with everything that can be read off the
    directory filled in: model-parallel size = number of ``reshard*.pt`` files, tokenizer files from their
    conventional names (``gpt2-unified.json``, else ``gpt2-vocab.json`` + ``gpt2-merges.txt``), checkpoint path
    ``<dir>/reshard.pt`` (reference: metaseq/scripts/convert_to_singleton.py:56-117)."""
    import glob

    from metaseq_b200 import options
    from metaseq_b200.dataclass.utils import convert_namespace_to_config

    mp = max(1, len(glob.glob(os.path.join(model_path, "reshard*.pt"))))
    unified = os.path.join(model_path, "gpt2-unified.json")
    merges, vocab = os.path.join(model_path, "gpt2-merges.txt"), os.path.join(model_path, "gpt2-vocab.json")
    if os.path.exists(unified):
        tokenizer_args = ["--hf-tokenizer", unified]
    else:
        tokenizer_args = ["--bpe-merges", merges, "--merges-filename", merges, "--bpe-vocab", vocab,
                          "--vocab-filename", vocab]
    argv = ["--model-parallel-size", str(mp), "--distributed-world-size", str(mp), "--ddp-backend", ddp_backend,
            "--task", "language_modeling", *tokenizer_args, "--bpe", "hf_byte_bpe",
            "--path", os.path.join(model_path, "reshard.pt"), "--checkpoint-shard-count", "1", "--use-sharded-state",
            model_path]
    parser = options.get_generation_parser()
    parser.set_defaults(lr_scheduler=None, criterion=None)
    cfg = convert_namespace_to_config(options.parse_args_and_arch(parser, input_args=argv))
    cfg.distributed_training.distributed_world_size = mp
    return cfg


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("location")
    ap.add_argument("--prefix", default="reshard")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    print(convert_to_singleton(a.location, a.prefix))


if __name__ == "__main__":
    main()
