"""Prompt loop on stdin against the same generator the hosted API uses (reference:
metaseq/cli/interactive_cli.py:44-125).  Rank 0 reads prompts and broadcasts the request; all
ranks run the generation."""
from __future__ import annotations

import os
import random
import sys

import torch

from metaseq_b200 import options
from metaseq_b200.dataclass.utils import convert_namespace_to_config
from metaseq_b200.hub_utils import GeneratorInterface
from metaseq_b200.parallel import utils as dist_utils
from metaseq_b200.service import constants as C
from metaseq_b200.service.utils import build_logger

logger = build_logger()


def input_loop():
    lines = []
    while True:
        try:
            line = input()
        except EOFError:
            if lines:
                return "\n".join(lines)
            raise KeyboardInterrupt
        if line.strip() == "":
            if lines:
                return "\n".join(lines)
            continue
        lines.append(line)


def worker_main(cfg, namespace_args=None):
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    generator = GeneratorInterface(cfg)
    generator.load_model()
    logger.info(f"loaded model {cfg.distributed_training.distributed_rank}")
    rank0 = not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0
    if rank0:
        logger.info("Model training complete! Enter a prompt followed by an empty line; Ctrl-D to quit.")
        while True:
            try:
                prompt = input_loop()
            except KeyboardInterrupt:
                break
            tokens = generator.encode_fn(prompt)
            request = {"inputs": [tokens], "max_tokens": [128], "temperature": 0.7, "top_p": 0.9, "n": 1,
                       "seed": random.randint(1, 20000)}
            if torch.distributed.is_initialized():
                dist_utils.broadcast_object(request, src_rank=0, group=dist_utils.get_global_group())
            out = generator.generate(**request)
            print(out[0][0]["text"], flush=True)
    else:
        while True:
            request = dist_utils.broadcast_object(None, src_rank=0, group=dist_utils.get_global_group())
            generator.generate(**request)


def cli_main():
    parser = options.get_generation_parser()
    flat = []
    for s in C.LAUNCH_ARGS:
        flat += s.split()
    args = options.parse_args_and_arch(parser, input_args=flat + sys.argv[1:])
    args.data = os.path.dirname(args.path)
    cfg = convert_namespace_to_config(args)
    dist_utils.call_main(cfg, worker_main, namespace_args=args)


if __name__ == "__main__":
    cli_main()
