"""Per-kernel timing against the measured roofline.

``python -m metaseq_b200.benchmark.kernels [--model opt-1.3b] [--out FILE]``

For every hot op of one decoder layer (and the logits / loss / optimizer ops)
this times the sm_100a kernel and the PyTorch/cuBLAS restatement of the same op
with CUDA events on the launching stream, after warm-up, flushing L2 between
iterations by writing a buffer larger than L2.  Fractions are reported "of
measured": the denominators are the copy bandwidth and cuBLAS bf16 throughput
recorded in ``MEASURED_PEAKS.json`` at the repository root (fallback 6.65 TB/s
and 1.59 PFLOP/s when the file is absent).

The reference ships only whole-model harnesses (metaseq/benchmark/generator.py,
``--benchmark`` in metaseq/launcher/opt_baselines.py:59-63); this per-op view is
what the roofline accounting needs.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch

from metaseq_b200.ops import functional as F
from metaseq_b200.ops import _lib

SHAPES = {
    "opt-125m": dict(D=768, H=12, FFN=3072, V=50272),
    "opt-1.3b": dict(D=2048, H=32, FFN=8192, V=50272),
    "opt-6.7b": dict(D=4096, H=32, FFN=16384, V=50272),
    "opt-30b": dict(D=7168, H=56, FFN=28672, V=50272),
}


def load_peaks():
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d["bf16_tflops"], tflops_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _FLUSH.fill_(1)


def time_op(fn, warmup=3, iters=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush_l2()
        # a bounded device-side delay (about a millisecond) lets the host enqueue fn() before the start event runs,
        # so an op with a long host path (allocations, tensor-map encoding) is not timed with the GPU idle
        torch.cuda._sleep(1_500_000)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2], times[0]


def time_graphed(fn, variants: int, launches: int = 24, dependent: bool = False):
    """Mean time in ms of ``fn(i)`` launched ``launches`` times from one CUDA graph, ``i`` cycling over ``variants``
    operand sets whose total size exceeds L2.  For kernels of a few microseconds an eager launch measures the
    launch path, not the kernel; this is also how the decode step runs them.  ``dependent``: capture with
    programmatic dependent launch, as the decode step does."""
    import contextlib

    for i in range(min(3, variants)):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with (F.dependent_launch() if dependent else contextlib.nullcontext()):
        with torch.cuda.graph(graph):
            for i in range(launches):
                fn(i % variants)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) / launches)
    times.sort()
    return times[len(times) // 2]


def _torch_top_p(lprobs, uniform):
    prev = F.get_backend()
    F.set_backend("torch")
    try:
        return F.sample_top_p(lprobs, 0.9, uniform)
    finally:
        F.set_backend(prev)


def with_backend(name, fn):
    def run():
        prev = F.get_backend()
        F.set_backend(name)
        try:
            return fn()
        finally:
            F.set_backend(prev)
    return run


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="opt-1.3b", choices=sorted(SHAPES))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--out", default=None)
    ap.add_argument("--only", default=None, help="comma-separated op-name prefixes")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gemm-variant", default="auto", choices=["auto", "1cta", "2cta"])
    ap.add_argument("--decode-batch", type=int, default=32, help="rows of the decode-step ops (--only decode)")
    ap.add_argument("--decode-cache", type=int, default=567, help="cached positions for the decode attention")
    args = ap.parse_args(argv)
    dt = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    F.set_gemm_variant(args.gemm_variant)
    cfg = SHAPES[args.model]
    D, H, FFN, V = cfg["D"], cfg["H"], cfg["FFN"], cfg["V"]
    B, T = args.batch, args.seq
    M = B * T
    d = D // H
    peaks = load_peaks()
    dev = "cuda"
    results = []

    def want(name):
        return args.only is None or any(name.startswith(p) for p in args.only.split(","))

    def report(name, flops, bytes_, fn_kernel, fn_torch):
        if not want(name):
            return
        med, best = time_op(fn_kernel, iters=args.iters)
        rec = dict(op=name, ms=round(med, 4), ms_best=round(best, 4))
        if flops:
            rec["tflops"] = round(flops / med / 1e9, 1)
            rec["frac_of_measured_gemm_peak"] = round(flops / med / 1e9 / peaks["tflops"], 3)
        if bytes_:
            rec["gbs"] = round(bytes_ / med / 1e6, 1)
            rec["frac_of_measured_hbm"] = round(bytes_ / med / 1e6 / peaks["hbm_gbs"], 3)
        if fn_torch is not None:
            tmed, _ = time_op(fn_torch, iters=args.iters)
            rec["torch_ms"] = round(tmed, 4)
            rec["speedup_vs_torch"] = round(tmed / med, 3)
        rec["peaks"] = peaks["source"]
        results.append(rec)
        print(json.dumps(rec), flush=True)

    x = torch.randn(M, D, device=dev, dtype=dt)
    # ---- GEMMs of one layer: forward (x W^T), dgrad (dy W), wgrad (dy^T x)
    for name, N, K in [("qkv", 3 * D, D), ("out_proj", D, D), ("fc1", FFN, D), ("fc2", D, FFN), ("logits", V, D)]:
        a = torch.randn(M, K, device=dev, dtype=dt)
        w = torch.randn(N, K, device=dev, dtype=dt) * 0.02
        dy = torch.randn(M, N, device=dev, dtype=dt)
        bias = torch.randn(N, device=dev, dtype=dt)
        out = torch.empty(M, N, device=dev, dtype=dt)
        dx = torch.empty(M, K, device=dev, dtype=dt)
        dw = torch.empty(N, K, device=dev, dtype=dt)
        fl = 2.0 * M * N * K
        report(f"gemm_fwd_{name}", fl, 0, lambda: F.gemm(a, w, bias=bias, out=out),
               lambda: torch.addmm(bias, a, w.t(), out=out))
        if name == "logits":
            # the same product with the softmax pieces of every row left by the epilogue, and the loss built on them
            report("gemm_rowstats_logits", fl, 0, lambda: F.gemm_with_row_stats(a, w), None)
            lg, st = F.gemm_with_row_stats(a, w)
            tgt_ce = torch.randint(0, N, (M,), device=dev)
            if st is not None:
                report("cross_entropy_from_row_stats", 0, 2.0 * M * N * 2,
                       lambda: F.cross_entropy_from_row_stats(lg, tgt_ce, 1, 1.0, st),
                       lambda: F.cross_entropy_fwd_bwd(lg, tgt_ce, 1, 1.0, True) if N * 2 <= 200 * 1024 else None)
            del lg, st
        report(f"gemm_dgrad_{name}", fl, 0, lambda: F.gemm(dy, w, b_mn=True, out=dx),
               lambda: torch.matmul(dy, w, out=dx))
        report(f"gemm_wgrad_{name}", fl, 0, lambda: F.gemm(dy, a, a_mn=True, b_mn=True, out=dw),
               lambda: torch.matmul(dy.t(), a, out=dw))
        del a, w, dy, out, dx, dw
    # ---- attention
    qkv = (torch.randn(B, T, 3 * D, device=dev) * 0.5).to(dt)
    k = qkv[..., 0:D].view(B, T, H, d)
    v = qkv[..., D:2 * D].view(B, T, H, d)
    q = qkv[..., 2 * D:].view(B, T, H, d)
    scale = d ** -0.5
    att_flops = 4.0 * B * H * T * T * d / 2

    def sdpa():
        return torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)

    if F.attn_head_dim_ok(d):
        report("attn_fwd", att_flops, 0, lambda: F.flash_attn_fwd(q, k, v, scale, True), sdpa)
        out, lse = F.flash_attn_fwd(q, k, v, scale, True)
        d_out = torch.randn_like(out)
        dqkv = torch.empty_like(qkv)
        dk = dqkv[..., 0:D].view(B, T, H, d)
        dv = dqkv[..., D:2 * D].view(B, T, H, d)
        dq = dqkv[..., 2 * D:].view(B, T, H, d)
        qg = q.detach().transpose(1, 2).requires_grad_(True)
        kg = k.detach().transpose(1, 2).requires_grad_(True)
        vg = v.detach().transpose(1, 2).requires_grad_(True)
        o_ref = torch.nn.functional.scaled_dot_product_attention(qg, kg, vg, is_causal=True)
        go = torch.randn_like(o_ref)

        def sdpa_bwd():
            torch.autograd.grad(o_ref, (qg, kg, vg), go, retain_graph=True)

        report("attn_bwd", 2.5 * att_flops, 0,
               lambda: F.flash_attn_bwd(q, k, v, out, d_out, lse, scale, True, dq, dk, dv), sdpa_bwd)
    # ---- memory-bound ops
    g = torch.ones(D, device=dev, dtype=dt)
    b = torch.zeros(D, device=dev, dtype=dt)
    report("layernorm_fwd", 0, 2.0 * M * D * 2, lambda: F.layer_norm_fwd(x, g, b, 1e-5),
           lambda: torch.nn.functional.layer_norm(x, (D,), g, b, 1e-5))
    y, mean, rstd = F.layer_norm_fwd(x, g, b, 1e-5)
    dy = torch.randn_like(x)
    report("layernorm_bwd", 0, 3.0 * M * D * 2, lambda: F.layer_norm_bwd(dy, x, mean, rstd, g), None)
    # with the residual-branch gradient added in the same pass, as the fused layer calls it
    report("layernorm_bwd_add", 0, 4.0 * M * D * 2, lambda: F.layer_norm_bwd(dy, x, mean, rstd, g, add=y), None)
    for name, width in (("qkv", 3 * D), ("fc1", FFN)):
        wide = torch.randn(M, width, device=dev, dtype=dt)
        db = torch.zeros(width, device=dev, dtype=dt)
        report(f"bias_grad_colsum_{name}", 0, 1.0 * M * width * 2, lambda: F.colsum(wide, out16=db, accumulate=True),
               lambda: torch.sum(wide, dim=0, dtype=torch.float32))
        del wide, db
    rows = min(M, 4096)
    logits = torch.randn(rows, V, device=dev, dtype=dt)
    tgt = torch.randint(0, V, (rows,), device=dev)
    report("cross_entropy_fwd_bwd", 0, 2.0 * rows * V * 2,
           lambda: F.cross_entropy_fwd_bwd(logits, tgt, 1, 1.0, True),
           with_backend("torch", lambda: F.cross_entropy_fwd_bwd(logits, tgt, 1, 1.0, True)))
    n = 12 * D * D + 13 * D
    n -= n % 8
    p = torch.randn(n, device=dev, dtype=dt)
    gr = torch.randn(n, device=dev, dtype=dt)
    m_ = torch.zeros(n, device=dev)
    v_ = torch.zeros(n, device=dev)
    acc = torch.zeros(1, device=dev)
    report("sumsq_layer_flat", 0, n * 2.0, lambda: F.sumsq(gr, acc, False), lambda: gr.float().pow(2).sum())
    kw = dict(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3)
    report("adamw_layer_flat", 0, n * (2 + 2 * 2 + 4 * 4.0), lambda: F.adamw_step(p, gr, m_, v_, **kw), None)
    # ---- decode step: few-row products and single-query attention, launched from a graph
    Bd, Sd = args.decode_batch, args.decode_cache
    if want("decode"):
        xd = torch.randn(Bd, max(D, FFN), device=dev, dtype=dt)
        for name, N, K in [("qkv", 3 * D, D), ("out_proj", D, D), ("fc1", FFN, D), ("fc2", D, FFN), ("logits", V, D)]:
            copies = max(2, int(300e6 / (N * K * 2)) + 1)
            ws = [torch.randn(N, K, device=dev, dtype=dt) * 0.02 for _ in range(copies)]
            outd = torch.empty(Bd, N, device=dev, dtype=dt)
            xin = xd[:, :K]
            rec = dict(op=f"decode_gemm_{name}", rows=Bd, N=N, K=K,
                       split=_lib.kernels().msq_gemm_skinny_split(N, K))
            for label, fn, dep in [("ms", lambda i: F.gemm(xin, ws[i], out=outd), False),
                                   ("ms_dependent_launch", lambda i: F.gemm(xin, ws[i], out=outd), True),
                                   ("cublas_ms", lambda i: torch.matmul(xin, ws[i].t(), out=outd), False)]:
                rec[label] = round(time_graphed(fn, copies, dependent=dep), 5)
            best = min(rec["ms"], rec["ms_dependent_launch"])
            rec["gbs"] = round(N * K * 2 / best / 1e6, 1)
            rec["frac_of_measured_hbm"] = round(rec["gbs"] / peaks["hbm_gbs"], 3)
            rec["peaks"] = peaks["source"]
            results.append(rec)
            print(json.dumps(rec), flush=True)
            del ws
        cap = -(-(Sd + 1) // 256) * 256
        copies = max(2, int(300e6 / (Bd * cap * D * 4)) + 1)
        caches = [(torch.randn(Bd, cap, D, device=dev, dtype=dt), torch.randn(Bd, cap, D, device=dev, dtype=dt))
                  for _ in range(copies)]
        qkv_d = torch.randn(Bd, 3 * D, device=dev, dtype=dt)
        length = torch.tensor([Sd], dtype=torch.int32, device=dev)
        ms = time_graphed(lambda i: F.decode_attn_step(qkv_d[:, 2 * D:], qkv_d[:, :D], qkv_d[:, D:2 * D], caches[i][0],
                                                       caches[i][1], length, H, scale, Sd), copies)
        nbytes = 2.0 * Bd * (Sd + 1) * D * 2
        rec = dict(op="decode_attn_step", batch=Bd, cached=Sd, ms=round(ms, 5), gbs=round(nbytes / ms / 1e6, 1),
                   frac_of_measured_hbm=round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 3), peaks=peaks["source"])
        results.append(rec)
        print(json.dumps(rec), flush=True)
        del caches
        # nucleus sampling over the full vocabulary (fp32 log-probabilities), against the sort-based restatement
        lps = [torch.log_softmax(torch.randn(Bd, V, device=dev) * 3, -1) for _ in range(4)]
        uni = torch.rand(Bd, device=dev)
        ms = time_graphed(lambda i: F.sample_top_p(lps[i], 0.9, uni), 4)
        tms = time_graphed(lambda i: _torch_top_p(lps[i], uni), 4)
        rec = dict(op="sample_top_p", rows=Bd, V=V, ms=round(ms, 5), torch_sort_ms=round(tms, 5),
                   speedup_vs_torch=round(tms / ms, 2))
        results.append(rec)
        print(json.dumps(rec), flush=True)
    bad = _lib.check_status(dev)
    summary = dict(model=args.model, batch=B, seq=T, dtype=args.dtype, peaks=peaks, kernel_status=bad,
                   device=torch.cuda.get_device_name(0))
    print(json.dumps(summary), flush=True)
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            for r in results:
                f.write(json.dumps(r) + "\n")
            f.write(json.dumps(summary) + "\n")


if __name__ == "__main__":
    main()
