"""Prefill and per-token decode latency of a random-init OPT model through the generation stack
(``SequenceGenerator`` -> model with KV cache), on one GPU.

    python -m metaseq_b200.benchmark.decode --arch opt_1_3b --batch 32 --prompt 512 --gen 128

Timing: CUDA events on the launching stream around whole ``generate`` calls, after warm-up calls.  The prefill
time is a call that generates one token; the decode time per token is the difference between a call generating
``--gen`` tokens and that call, divided by ``gen - 1``.  ``--kernel-backend torch`` runs the same model on
PyTorch ops (library attention, cuBLAS) for comparison."""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from metaseq_b200 import options, tasks
from metaseq_b200.dataclass.utils import convert_namespace_to_config
from metaseq_b200.sequence_generator import SequenceGenerator
from metaseq_b200.ops import _lib
from metaseq_b200.ops import functional as F


def init_tensor_parallel() -> int:
    """Under ``torchrun`` every rank holds a 1 / WORLD_SIZE slice of the model (tensor parallelism)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        import torch.distributed as dist

        from metaseq_b200.parallel import mpu

        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        mpu.initialize_model_parallel(world)
        mpu.model_parallel_cuda_manual_seed(1)
    return world


def build(arch: str, max_positions: int, tp: int = 1):
    parser = options.get_training_parser()
    ns = options.parse_args_and_arch(parser, input_args=[
        "--task", "dummy_lm", "--dict-size", "50268", "--tokens-per-sample", str(max_positions), "--batch-size", "1",
        "--arch", arch, "--criterion", "vocab_parallel_cross_entropy", "--optimizer", "adam", "--lr", "1e-3",
        "--memory-efficient-fp16", "--tensor-parallel-init-model-on-gpu", "--distributed-world-size", str(tp),
        "--model-parallel-size", str(tp), "--dropout", "0.0", "--attention-dropout", "0.0"])
    cfg = convert_namespace_to_config(ns)
    task = tasks.setup_task(cfg.task)
    torch.manual_seed(1)
    model = task.build_model(cfg.model).half().cuda().eval()
    model.make_generation_fast_()
    return cfg, task, model


def timed(fn, warmup, repeats):
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(repeats):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        samples.append(s.elapsed_time(e))
    return float(np.median(samples))


def measure(arch: str, batch: int, prompt: int, gen: int, warmup: int = 2, repeats: int = 3, tp: int = 1,
            top_p: float = -1.0, decode_graph: bool = True, kernel_backend: str = "auto") -> dict:
    """Builds the random-init model (this rank's slice under tensor parallelism; the process group and the
    model-parallel groups must exist already) and times whole ``generate`` calls.  Returns the record that
    ``main`` prints; under tensor parallelism the times are the slowest rank's."""
    cfg, task, model = build(arch, prompt + gen + 8, tp)
    rng = np.random.RandomState(0)
    prompts = torch.from_numpy(rng.randint(100, 50000, size=(batch, prompt))).cuda()
    sample = {"net_input": {"src_tokens": prompts}}

    def call(n_new):
        total = prompt + n_new
        sg = SequenceGenerator([model], task.target_dictionary, beam_size=1, max_len_b=total, min_len=total,
                               temperature=1.0, topp=top_p, decode_graph=decode_graph)
        with torch.no_grad():
            return sg.generate([model], sample)

    _lib.reset_launch_count()
    t1 = timed(lambda: call(1), warmup, repeats)
    tn = timed(lambda: call(gen), 1, repeats)
    if tp > 1:
        import torch.distributed as dist

        worst = torch.tensor([t1, tn], device="cuda")
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)  # the slowest rank's device time
        t1, tn = worst.tolist()
    per_tok = (tn - t1) / max(1, gen - 1)
    out = dict(metric="decode_ms_per_token", arch=arch, batch=batch, prompt_len=prompt, gen_len=gen,
               prefill_ms=round(t1, 2), total_ms=round(tn, 2), decode_ms_per_token=round(per_tok, 3),
               decode_tokens_per_s=round(batch / per_tok * 1e3, 1), kernel_backend=kernel_backend,
               kernel_launches=_lib.launch_count(), kernel_status=_lib.check_status(torch.device("cuda")),
               tensor_parallel=tp, decode_graph=decode_graph, top_p=top_p,
               dtype="fp16", data="synthetic uniform token ids, random-init weights")
    del model
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="opt_1_3b")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--gen", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--kernel-backend", default="auto", choices=["auto", "torch"])
    ap.add_argument("--no-decode-graph", action="store_true", help="decode through the module tree")
    ap.add_argument("--top-p", type=float, default=-1.0, help="nucleus sampling mass; <= 0 decodes greedily")
    ap.add_argument("--graph-replays", type=int, default=0,
                    help="instead of whole generate calls: one prefill, then this many replays of the captured "
                         "decode step, timed together (the workload for a per-kernel launch list)")
    args = ap.parse_args(argv)
    F.set_backend(args.kernel_backend)
    tp = init_tensor_parallel()
    rank0 = int(os.environ.get("RANK", "0")) == 0
    if args.graph_replays > 0:
        from metaseq_b200.models.decode_step import GraphedDecodeStep

        cfg, task, model = build(args.arch, args.prompt + args.gen + 8, tp)
        rng = np.random.RandomState(0)
        prompts = torch.from_numpy(rng.randint(100, 50000, size=(args.batch, args.prompt))).cuda()
        assert GraphedDecodeStep.supported(model.decoder, args.batch), "the graphed step needs the kernel backend"
        runner = GraphedDecodeStep.for_decoder(model.decoder, args.batch, args.prompt + 2 * args.graph_replays + 8)
        with torch.no_grad():
            model(prompts, incremental_state=runner.new_state())
            runner.begin(prompts)
            nxt = prompts[:, -1].clone()
            runner.step(nxt)  # captures
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(args.graph_replays):
                runner.step(nxt)
            e.record()
            torch.cuda.synchronize()
            # the captured part alone (under tensor parallelism the embedding and the projection are outside it)
            s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s2.record()
            for _ in range(args.graph_replays):
                runner.graph.replay()
            e2.record()
            torch.cuda.synchronize()
        if rank0:
            print(json.dumps(dict(metric="decode_graph_step_ms", arch=args.arch, batch=args.batch, cached=args.prompt,
                                  replays=args.graph_replays, tensor_parallel=tp,
                                  ms_per_replay=round(s.elapsed_time(e) / args.graph_replays, 4),
                                  ms_graph_only=round(s2.elapsed_time(e2) / args.graph_replays, 4),
                                  kernel_status=_lib.check_status(torch.device("cuda")))), flush=True)
        return
    out = measure(args.arch, args.batch, args.prompt, args.gen, args.warmup, args.repeats, tp, args.top_p,
                  not args.no_decode_graph, args.kernel_backend)
    if rank0:
        print(json.dumps(out), flush=True)
    if tp > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
