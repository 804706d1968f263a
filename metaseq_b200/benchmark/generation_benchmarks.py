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


# ---- the reference's fixed-prompt benchmark: one forward pass over 1000 copies of a sentence per released model
PROMPTS = ["Paris is the capital of France and it"] * 1000
_RELEASE = "https://dl.fbaipublicfiles.com/opt/v1_20220502"
_PARTS = {"125m": 2, "1.3b": 2, "2.7b": 4, "6.7b": 2, "13b": 2, "30b": 2}
LINKS_TO_DATA = {name: [f"{_RELEASE}/{name}/reshard-model_part-{i}.pt" for i in range(n)] for name, n in _PARTS.items()}
LINKS_TO_DATA["66b"] = [f"{_RELEASE}/66b/reshard-model_part-{i}-shard0.pt" for i in range(8)]
LINKS_TO_DATA["dependencies"] = ["http://dl.fbaipublicfiles.com/metaseq_benchmark_dependencies.tar.gz"]


def load_mp_model_and_run_eval(cfg, model_path: str = "", prompts=None, **_unused):
    """On every rank: tokenize the prompts, load this rank's model part, score all prompts in one forward pass.
    Returns the seconds (tokenization + forward) of every rank (reference:
    metaseq/scripts/generation_benchmarks.py:79-142)."""
    import time

    from metaseq_b200.hub_utils import setup_vocab_and_merges, tensorize_input

    prompts = PROMPTS if prompts is None else prompts
    on_gpu = torch.cuda.is_available() and not cfg.common.cpu
    _, _, tokenizer = setup_vocab_and_merges(model_path)
    t0 = time.perf_counter()
    ids = torch.cat([tensorize_input(tokenizer, p) for p in prompts])
    if on_gpu:
        ids = ids.cuda()
    tokenize_s = time.perf_counter() - t0
    generator = GeneratorInterface(cfg)
    model = generator.load_model()[0].eval()
    with torch.no_grad():
        if on_gpu:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            model(ids)
            end.record()
            torch.cuda.synchronize()
            forward_s = start.elapsed_time(end) / 1e3
        else:
            t0 = time.perf_counter()
            model(ids)
            forward_s = time.perf_counter() - t0
    mine = torch.tensor([tokenize_s + forward_s], device=ids.device)
    if not torch.distributed.is_initialized():
        return [mine]
    times = [torch.zeros_like(mine) for _ in range(dist_utils.get_global_world_size())]
    torch.distributed.all_gather(times, mine, group=dist_utils.get_global_group())
    return times


def generation_statistics(model_path: str, prompts=None, cpu: bool = False):
    """Prints the mean time over ranks and characters of prompt per second, as the reference does (it calls them
    words)."""
    from metaseq_b200.checkpoint.convert_to_singleton import create_generation_config_with_defaults

    cfg = create_generation_config_with_defaults(model_path)
    cfg.common.cpu = cfg.common.cpu or cpu
    prompts = PROMPTS if prompts is None else prompts
    times = dist_utils.call_main(cfg, load_mp_model_and_run_eval, model_path=model_path, prompts=prompts)
    mean_s = float(sum(float(t) for t in times) / len(times))
    print("Total generation time " + str(mean_s))
    print("Words per second : " + str(len(prompts[0]) * len(prompts) / mean_s))
    return mean_s


def download_data(key: str, into: str = "."):
    """Fetches the tokenizer files and the released checkpoint parts of ``key`` into ``<into>/dependencies``
    (needs network access)."""
    import tarfile
    import urllib.request

    if key not in LINKS_TO_DATA or key == "dependencies":
        raise AssertionError(f"You passed model name {key}. Please make sure that model name is in "
                             f"{[k for k in LINKS_TO_DATA if k != 'dependencies']}")
    import os

    for url in LINKS_TO_DATA["dependencies"]:
        archive = os.path.join(into, "dependencies.tar.gz")
        urllib.request.urlretrieve(url, archive)
        with tarfile.open(archive) as tar:
            tar.extractall(into)
    for url in LINKS_TO_DATA[key]:
        urllib.request.urlretrieve(url, os.path.join(into, "dependencies", url.rsplit("/", 1)[1]))


def cleanup_data(into: str = "."):
    import os
    import shutil

    shutil.rmtree(os.path.join(into, "dependencies"), ignore_errors=True)
    if os.path.exists(os.path.join(into, "dependencies.tar.gz")):
        os.remove(os.path.join(into, "dependencies.tar.gz"))


def cli_main():
    if any(a.startswith("--model_name") or a.startswith("--model-name") for a in sys.argv[1:]):
        import argparse

        ap = argparse.ArgumentParser(description="fixed-prompt benchmark over released models (downloads them)")
        ap.add_argument("--model_name", "--model-name", nargs="+", required=True)
        names = ap.parse_args().model_name
        for key in names:
            print("Now running generation benchmarks for " + str(key))
            download_data(key)
            generation_statistics(model_path="./dependencies")
            cleanup_data()
        return 0

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
