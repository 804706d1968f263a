"""Sweeps generation settings (batch size x prompt length x generated length x beam) over one loaded model and
prints a table of latency and throughput (reference: metaseq/scripts/generation_benchmarks.py).

    python -m metaseq_b200.benchmark.generation_benchmarks --path <ckpt> \
        --batch-sizes 1,8,32 --prompt-lengths 32,512 --gen-lengths 32,128 --beams 1

Each cell: ``--warmup`` untimed calls, then ``--repeats`` calls timed with CUDA events; tokens/s counts generated
tokens only."""
from __future__ import annotations

import itertools
import json
import logging
import sys

import numpy as np
import torch

from metaseq_b200 import options
from metaseq_b200.dataclass.utils import convert_namespace_to_config
from metaseq_b200.hub_utils import GeneratorInterface
from metaseq_b200.parallel import utils as dist_utils

logger = logging.getLogger(__name__)


def _ints(s):
    return [int(x) for x in str(s).split(",") if x]


def time_cell(generator, batch, prompt_len, gen_len, beam, warmup, repeats, vocab_hi=50000):
    def call():
        prompts = np.random.randint(100, vocab_hi, size=(batch, prompt_len)).tolist()
        return generator.generate(prompts, min_tokens=[gen_len] * batch, max_tokens=[gen_len] * batch, n=beam,
                                  temperature=1.0, top_p=0.9)

    for _ in range(warmup):
        call()
    samples = []
    for _ in range(repeats):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        call()
        e.record()
        torch.cuda.synchronize()
        samples.append(s.elapsed_time(e))
    ms = float(np.median(samples))
    return dict(batch=batch, prompt_len=prompt_len, gen_len=gen_len, beam=beam, ms=round(ms, 2),
                ms_per_token=round(ms / gen_len, 3), gen_tokens_per_s=round(batch * beam * gen_len / ms * 1e3, 1))


def main(cfg, grid=None, warmup=2, repeats=5, out=None):
    generator = GeneratorInterface(cfg)
    generator.load_model()
    rows = []
    for b, p, g, k in itertools.product(*grid):
        row = time_cell(generator, b, p, g, k, warmup, repeats)
        rows.append(row)
        if not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0:
            print(json.dumps(row), flush=True)
    if out and (not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0):
        with open(out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


def cli_main():
    parser = options.get_generation_parser()
    parser.add_argument("--batch-sizes", default="1,8")
    parser.add_argument("--prompt-lengths", default="32,256")
    parser.add_argument("--gen-lengths", default="32")
    parser.add_argument("--beams", default="1")
    parser.add_argument("--warmup", type=int, default=2)
    parser.add_argument("--repeats", type=int, default=5)
    parser.add_argument("--out", default=None)
    args = options.parse_args_and_arch(parser)
    cfg = convert_namespace_to_config(args)
    grid = (_ints(args.batch_sizes), _ints(args.prompt_lengths), _ints(args.gen_lengths), _ints(args.beams))
    dist_utils.call_main(cfg, main, grid=grid, warmup=args.warmup, repeats=args.repeats, out=args.out)


if __name__ == "__main__":
    sys.exit(cli_main())
