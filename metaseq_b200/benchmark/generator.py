"""Generation latency benchmark: loads a checkpoint through ``GeneratorInterface`` and times ``generate`` on
random prompts of ``--max-source-positions`` tokens producing ``--max-target-positions`` tokens
(reference: metaseq/benchmark/generator.py:35-136).

    python -m metaseq_b200.benchmark.generator --path <ckpt> --batch-size 8 \
        --max-source-positions 128 --max-target-positions 128 [--profile]

Latency is measured with CUDA events on the launching stream after warm-up runs; peak memory is summed over
ranks.  ``--profile`` writes a torch profiler trace (schedule: skip 5, wait 5, warm up 5, record 2)."""
from __future__ import annotations

import logging
import random
import socket
from typing import Tuple

import numpy as np
import torch

from metaseq_b200 import options
from metaseq_b200.dataclass.utils import convert_namespace_to_config
from metaseq_b200.hub_utils import GeneratorInterface
from metaseq_b200.parallel import utils as dist_utils

logger = logging.getLogger(__name__)
WARMUP_STEPS = 5
NUM_REPEATS = 5


def _random_prompts(batch_size: int, length: int):
    return np.random.randint(100, 50000, size=(batch_size, length)).tolist()


def _one_call(generator, cfg, batch_size, input_length, output_length):
    return generator.generate(inputs=_random_prompts(batch_size, input_length), max_tokens=[output_length] * batch_size,
                              temperature=cfg.generation.temperature, n=cfg.generation.beam, top_p=0.9)


def benchmark(generator, cfg, batch_size: int, input_length: int, output_length: int) -> Tuple[np.ndarray, float]:
    times = []
    for _ in range(NUM_REPEATS):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        _one_call(generator, cfg, batch_size, input_length, output_length)
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    peak = torch.tensor(float(torch.cuda.memory_stats()["allocated_bytes.all.peak"]), device="cuda")
    if torch.distributed.is_initialized():
        torch.distributed.all_reduce(peak)
    return np.array(times), float(peak.item())


def profile(generator, cfg, batch_size: int, input_length: int, output_length: int, out_dir: str = "traces") -> None:
    from torch.profiler import ProfilerActivity, schedule, tensorboard_trace_handler

    rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
    handler = tensorboard_trace_handler(dir_name=out_dir, worker_name=f"{socket.gethostname()}_{rank}", use_gzip=True)
    with torch.profiler.profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], profile_memory=True,
                                record_shapes=True, schedule=schedule(skip_first=5, wait=5, warmup=5, active=2, repeat=1),
                                on_trace_ready=handler, with_stack=True) as prof:
        for _ in range(17):
            _one_call(generator, cfg, batch_size, input_length, output_length)
            prof.step()


def main(cfg, do_profile: bool = False) -> None:
    torch.manual_seed(random.randint(1, 20000))
    logger.info("Instantiating a generator interface and loading a model")
    generator = GeneratorInterface(cfg)
    generator.load_model()
    batch_size = cfg.dataset.batch_size
    input_length = cfg.task.max_source_positions
    output_length = cfg.task.max_target_positions
    logger.info("Running warm-up steps before benchmarking")
    for _ in range(WARMUP_STEPS):
        generator.generate(_random_prompts(batch_size, input_length), max_tokens=[output_length] * batch_size)
    logger.info(f"Benchmarking with batch size {batch_size}, input length {input_length}, and output length {output_length}")
    if do_profile:
        profile(generator, cfg, batch_size, input_length, output_length)
        return
    elapsed, peak = benchmark(generator, cfg, batch_size, input_length, output_length)
    if not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0:
        print(f"Latency: {elapsed.mean():.4f} +/- {elapsed.std():.4f} ms")
        print(f"Peak memory usage: {peak / 1024 ** 3:.4f} GB")


def cli_main():
    parser = options.get_generation_parser()
    if not any("--profile" in a.option_strings for a in parser._actions):  # the common options already carry it
        parser.add_argument("--profile", action="store_true", help="record a profiler trace instead of timing")
    args = options.parse_args_and_arch(parser)
    cfg = convert_namespace_to_config(args)
    dist_utils.call_main(cfg, main, do_profile=getattr(args, "profile", False))


if __name__ == "__main__":
    cli_main()
