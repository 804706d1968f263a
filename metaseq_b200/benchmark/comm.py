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
    ap.add_argument("--transport", default="ce", choices=["ce", "sm"])
    args = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from metaseq_b200.ops import _lib
    from metaseq_b200.parallel.symm import PeerComm

    numel = int(args.unit_mb * 1e6 / 2) // (8 * world) * (8 * world)
    comm = PeerComm(dist.group.WORLD, dev, heap_bytes=4 * numel * 2 + (64 << 20), transport=args.transport)
    full = comm.alloc_full(numel, torch.float16)
    shard_in = torch.randn(numel // world, device=dev, dtype=torch.float16)
    grad = torch.randn(numel, device=dev, dtype=torch.float16)
    shard_out = torch.empty(numel // world, device=dev, dtype=torch.float16)
    ref_full = torch.empty(numel, device=dev, dtype=torch.float16)
    results = []

    def rec(op, ms, nccl_ms, bus_bytes):
        r = dict(op=op, n_gpus=world, ms=round(ms, 4), nccl_ms=round(nccl_ms, 4), speedup_vs_nccl=round(nccl_ms / ms, 3),
                 bus_gbs=round(bus_bytes / ms / 1e6, 1), frac_of_measured_nvlink=round(bus_bytes / ms / 1e6 / NVLINK_GBS, 3))
        results.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    moved = numel * 2 * (world - 1) / world  # bytes each GPU sends (and receives)
    rec("fsdp_unit_all_gather",
        _time(lambda: comm.all_gather(full, shard_in), args.iters),
        _time(lambda: dist.all_gather_into_tensor(ref_full, shard_in), args.iters), moved)
    rec("fsdp_unit_reduce_scatter_fp32sum_unscale_norm",
        _time(lambda: comm.reduce_scatter(shard_out, grad, key=full, scale=1.0 / world, accumulate_norm=True), args.iters),
        _time(lambda: dist.reduce_scatter_tensor(shard_out, grad), args.iters), moved)
    for nbytes in (16 << 10, 256 << 10, 1 << 20):
        x = torch.randn(nbytes // 2, device=dev, dtype=torch.float16)
        y = x.clone()
        nccl = _time(lambda: dist.all_reduce(y), args.iters)
        rec(f"all_reduce_peer_slots_{nbytes >> 10}KiB", _time(lambda: comm.all_reduce(x, use_multicast=False), args.iters), nccl,
            2 * nbytes * (world - 1) / world)
        if comm.heap.multicast_ptr:
            rec(f"all_reduce_in_switch_{nbytes >> 10}KiB", _time(lambda: comm.all_reduce(x, use_multicast=True), args.iters), nccl,
                2 * nbytes * (world - 1) / world)
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
