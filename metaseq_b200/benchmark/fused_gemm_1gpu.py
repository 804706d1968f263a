"""The communication-fused GEMM variants on one GPU, for profiling with tools that cannot follow several ranks.

The peers are emulated by local buffers: the flag-polling GEMM (`msq_gemm2_ready`) reads a weight whose arrival
flags are all already published (so the run shows the cost of polling, not of waiting), and the scattering GEMM
(`msq_gemm2_scatter`) stores the row blocks of its result into `--world` local slot buffers instead of peer memory.
Both are timed against the plain GEMM of the same shape with CUDA events (L2 flushed between iterations).

    python -m metaseq_b200.benchmark.fused_gemm_1gpu [--m 16384 --n 2048 --k 8192 --world 8]
"""
from __future__ import annotations

import argparse
import ctypes
import json

import torch

from metaseq_b200.benchmark.kernels import load_peaks, time_op
from metaseq_b200.ops import _lib
from metaseq_b200.ops import functional as F


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    M, N, K, W = args.m, args.n, args.k, args.world
    dev = torch.device("cuda")
    peaks = load_peaks()
    a = torch.randn(M, K, device=dev, dtype=torch.float16)
    w = torch.randn(N, K, device=dev, dtype=torch.float16) * 0.02
    out = torch.empty(M, N, device=dev, dtype=torch.float16)
    lib = _lib.kernels()
    status = _lib.ptr(_lib.status_word(dev))
    flops = 2.0 * M * N * K

    def rec(name, ms, base=None):
        r = dict(op=name, M=M, N=N, K=K, ms=round(ms, 4), tflops=round(flops / ms / 1e9, 1),
                 frac_of_measured_gemm_peak=round(flops / ms / 1e9 / peaks["tflops"], 3))
        if base:
            r["vs_plain_gemm"] = round(base / ms, 3)
        print(json.dumps(r), flush=True)

    plain, _ = time_op(lambda: F.gemm(a, w, out=out), iters=args.iters)
    rec("gemm_plain", plain)

    # flag-polling consumer: the weight is cut into W shards of 2 MiB chunks, all flags already at the epoch
    shard_bytes = N * K * 2 // W
    chunk = min(2 << 20, shard_bytes)
    chunks = (shard_bytes + chunk - 1) // chunk
    flags = torch.full((W * chunks,), 7, dtype=torch.int32, device=dev)
    desc = _lib.GemmReady(flags.data_ptr(), 0, shard_bytes, chunk, chunks, -1, 7, 0)

    def ready():
        rc = lib.msq_gemm2_ready(_lib.ptr(a), _lib.ptr(w), _lib.ptr(out), M, N, K, K, K, N, 0, 0, 0, None, None, 0, None, 0,
                                 0, 0, 0, 0, status, _lib.stream_ptr(), ctypes.byref(desc))
        _lib.check_rc(rc, "msq_gemm2_ready")

    t, _ = time_op(ready, iters=args.iters)
    rec("gemm_flag_polling_consumer", t, plain)

    # scattering producer: row block r goes to slot buffer r
    rows = M // W
    slots = [torch.empty(rows, N, device=dev, dtype=torch.float16) for _ in range(W)]
    dst = (ctypes.c_void_p * W)(*[s.data_ptr() for s in slots])

    def scatter():
        rc = lib.msq_gemm2_scatter(_lib.ptr(a), _lib.ptr(w), M, N, K, K, K, N, 0, 0, 0, dst, W, rows, 0, status,
                                   _lib.stream_ptr())
        _lib.check_rc(rc, "msq_gemm2_scatter")

    t, _ = time_op(scatter, iters=args.iters)
    rec("gemm_row_scatter_producer", t, plain)
    ref = (a[:256].float() @ w.float().t())
    err = (slots[0][:256].float() - ref).abs().max().item() / ref.abs().max().item()
    print(json.dumps(dict(check_rel_err=round(err, 5), kernel_status=_lib.check_status(dev))), flush=True)


if __name__ == "__main__":
    main()
