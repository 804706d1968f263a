"""Peer-memory collectives against NCCL, timed on the device.

``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m metaseq_b200.benchmark.comm``

For the all-gather and reduce-scatter of one FSDP unit and for small all-reduces this times the
kernels of ``csrc/comm_sm100.cu`` and the NCCL collective on the same buffers with CUDA events on the
launching stream (warm-up first, a barrier before each timed call), takes the maximum over ranks and
reports bus bandwidth against the measured NVLink peer-copy rate (770 GB/s per direction per GPU).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    t = torch.tensor([times[len(times) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--unit-mb", type=float, default=100.7, help="gathered size of one FSDP unit in MB (OPT-1.3B layer)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default=None)
    ap.add_argument("--transport", default="all", choices=["all", "ce", "sm", "mm"],
                    help="bulk transport of the all-gather / reduce-scatter: peer DMA (ce), store kernels (sm), "
                         "through NVSwitch with multimem (mm), or each of them in turn (all)")
    ap.add_argument("--decode-dim", type=int, default=4096, help="model width for the decode GEMM + all-reduce timing")
    ap.add_argument("--decode-rows", type=int, default=32)
    args = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from metaseq_b200.ops import _lib
    from metaseq_b200.parallel.symm import PeerComm

    numel = int(args.unit_mb * 1e6 / 2) // (8 * world) * (8 * world)
    shard_in = torch.randn(numel // world, device=dev, dtype=torch.float16)
    grad_src = torch.randn(numel, device=dev, dtype=torch.float16)
    shard_out = torch.empty(numel // world, device=dev, dtype=torch.float16)
    ref_full = torch.empty(numel, device=dev, dtype=torch.float16)
    ref_shard = torch.empty(numel // world, device=dev, dtype=torch.float16)
    results = []

    def rec(op, ms, nccl_ms, bus_bytes):
        r = dict(op=op, n_gpus=world, ms=round(ms, 4), nccl_ms=round(nccl_ms, 4), speedup_vs_nccl=round(nccl_ms / ms, 3),
                 bus_gbs=round(bus_bytes / ms / 1e6, 1), frac_of_measured_nvlink=round(bus_bytes / ms / 1e6 / NVLINK_GBS, 3))
        results.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    moved = numel * 2 * (world - 1) / world  # bytes each GPU sends (and receives)
    nccl_ag = _time(lambda: dist.all_gather_into_tensor(ref_full, shard_in), args.iters)
    nccl_rs = _time(lambda: dist.reduce_scatter_tensor(ref_shard, grad_src), args.iters)
    ref_shard.div_(world)
    comm = None
    for transport in (["ce", "sm", "mm"] if args.transport == "all" else [args.transport]):
        comm = PeerComm(dist.group.WORLD, dev, heap_bytes=4 * numel * 2 + (64 << 20), transport=transport)
        if transport == "mm" and not comm.heap.multicast_ptr:
            if rank == 0:
                print(json.dumps(dict(op="transport_mm", skipped="no multicast mapping")), flush=True)
            continue
        full = comm.alloc_full(numel, torch.float16)
        grad = comm.alloc_symmetric(numel, torch.float16) if comm.pulls_gradients else torch.empty_like(grad_src)
        grad.copy_(grad_src)
        torch.cuda.synchronize()
        dist.barrier()
        ag = _time(lambda: comm.all_gather(full, shard_in), args.iters)
        ag_err = float((full.float() - ref_full.float()).abs().max())
        rec(f"fsdp_unit_all_gather[{comm.ag_transport}]", ag, nccl_ag, moved)
        results[-1]["max_abs_diff_vs_nccl"] = ag_err

        def rs():
            comm.reduce_scatter(shard_out, grad, key=full, scale=1.0 / world, accumulate_norm=True)
            if comm.pulls_gradients:
                comm.barrier()  # as FSDP does once per backward: sources may be overwritten afterwards

        t_rs = _time(rs, args.iters)
        rs_err = float((shard_out.float() - ref_shard.float()).abs().max())
        rec(f"fsdp_unit_reduce_scatter_fp32sum_unscale_norm[{comm.rs_transport}]", t_rs, nccl_rs, moved)
        results[-1]["max_abs_diff_vs_nccl"] = rs_err
        if rank == 0:
            print(json.dumps(dict(check=transport, all_gather_max_abs_diff=ag_err, reduce_scatter_max_abs_diff=rs_err)),
                  flush=True)
    for nbytes in (16 << 10, 256 << 10, 1 << 20):
        x = torch.randn(nbytes // 2, device=dev, dtype=torch.float16)
        y = x.clone()
        nccl = _time(lambda: dist.all_reduce(y), args.iters)
        rec(f"all_reduce_peer_slots_{nbytes >> 10}KiB", _time(lambda: comm.all_reduce(x, use_multicast=False), args.iters), nccl,
            2 * nbytes * (world - 1) / world)
        if comm.heap.multicast_ptr:
            rec(f"all_reduce_in_switch_{nbytes >> 10}KiB", _time(lambda: comm.all_reduce(x, use_multicast=True), args.iters), nccl,
                2 * nbytes * (world - 1) / world)
    # ---- decode: few-row GEMM fused with the sum over ranks, launched from a graph, against the same product
    # without the exchange and against the product followed by an NCCL all-reduce
    from metaseq_b200.ops import functional as F
    from metaseq_b200.parallel.symm import DecodeReduce

    D, rows = args.decode_dim, args.decode_rows
    red = DecodeReduce(dist.group.WORLD, dev, 64, D, torch.float16)
    lib = _lib.kernels()
    shapes = [("out_proj", D // world), ("fc2", 4 * D // world)]
    split = min(lib.msq_gemm_skinny_split(D, k) for _, k in shapes)
    res = torch.randn(rows, D, device=dev, dtype=torch.float16)
    for name, K in shapes:
        copies = max(2, int(300e6 / (D * K * 2)) + 1)
        ws = [torch.randn(D, K, device=dev, dtype=torch.float16) * 0.02 for _ in range(copies)]
        x = torch.randn(rows, K, device=dev, dtype=torch.float16)
        launches = 24  # even: the staging halves keep alternating across replays

        def graphed(fn, dependent):
            import contextlib

            for i in range(2):
                fn(i)
            torch.cuda.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with (F.dependent_launch() if dependent else contextlib.nullcontext()):
                with torch.cuda.graph(g):
                    for i in range(launches):
                        fn(i % copies)
            return _time(g.replay, args.iters) / launches

        plain = graphed(lambda i: F.gemm(x, ws[i], residual=res), True)
        fused = graphed(lambda i: red.gemm_all_reduce(x, ws[i], residual=res, split=split), True)
        fused_nodep = graphed(lambda i: red.gemm_all_reduce(x, ws[i], residual=res, split=split), False)

        def gemm_then_nccl(i):
            y = F.gemm(x, ws[i])
            dist.all_reduce(y)
            return y.add_(res)

        for i in range(3):
            gemm_then_nccl(i)
        nccl = _time(lambda: [gemm_then_nccl(i % copies) for i in range(launches)], args.iters) / launches
        r = dict(op=f"decode_gemm_allreduce_{name}", n_gpus=world, rows=rows, N=D, K_local=K, cluster=split,
                 ms=round(fused, 5), ms_ordinary_launch=round(fused_nodep, 5), gemm_only_ms=round(plain, 5),
                 gemm_then_nccl_eager_ms=round(nccl, 5), exchange_bytes=rows * D * 2 * (world - 1))
        results.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)
        del ws
    bad = _lib.check_status(dev)
    if rank == 0:
        summary = dict(provider=comm.heap.provider, transport=args.transport, multicast=bool(comm.heap.multicast_ptr), kernel_status=bad,
                       unit_bytes=numel * 2, device=torch.cuda.get_device_name(local))
        print(json.dumps(summary), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as f:
                for r in results:
                    f.write(json.dumps(r) + "\n")
                f.write(json.dumps(summary) + "\n")
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
