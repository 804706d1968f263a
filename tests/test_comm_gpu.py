"""Peer-memory collectives against NCCL / plain PyTorch references, run as one process per GPU.

Needs at least two GPUs; on a single-GPU machine the tests are skipped."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, provider, transport, results):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from metaseq_b200.ops import _lib
        from metaseq_b200.parallel.symm import PeerComm

        dev = torch.device("cuda", rank)
        comm = PeerComm(dist.group.WORLD, dev, heap_bytes=512 << 20, chunk_bytes=1 << 18, provider=provider,
                        transport=transport)
        for _ in range(3):
            comm.barrier()
        torch.cuda.synchronize()
        # ---- all-gather (several epochs, ragged last chunk)
        numel = world * (3 * (1 << 17) + 8 * 13)
        full = comm.alloc_full(numel, torch.float16)
        for step in range(3):
            g = torch.Generator(device=dev).manual_seed(100 * step + rank)
            local = torch.randn(numel // world, device=dev, dtype=torch.float16, generator=g)
            ref = torch.empty(numel, device=dev, dtype=torch.float16)
            dist.all_gather_into_tensor(ref, local)
            comm.all_gather(full, local, stream=torch.cuda.Stream() if step == 1 else None)
            torch.cuda.synchronize()
            assert torch.equal(full, ref), f"all_gather mismatch at step {step}"
            dist.barrier()
        # ---- all-gather consumed by a GEMM that polls the arrival flags per tile (fused all-gather -> GEMM)
        from metaseq_b200.ops import functional as F

        Nw, Kw, Mx = 1024 * world, 512, 1024
        fullw = comm.alloc_full(Nw * Kw, torch.float16)
        handle = comm.ready_handle(fullw)
        wview = fullw.view(Nw, Kw)
        x = torch.randn(Mx, Kw, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(5))
        dyv = torch.randn(Mx, Nw, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(6))
        side = torch.cuda.Stream()
        for step in range(4):
            g = torch.Generator(device=dev).manual_seed(1000 + 10 * step + rank)
            local = torch.randn(Nw * Kw // world, device=dev, dtype=torch.float16, generator=g) * 0.05
            ref_w = torch.empty(Nw * Kw, device=dev, dtype=torch.float16)
            dist.all_gather_into_tensor(ref_w, local)
            ref_w = ref_w.view(Nw, Kw)
            torch.cuda.synchronize()
            dist.barrier()
            comm.all_gather_many([(fullw, local)], side)   # peer copies in flight on the side stream
            handle.active = True
            if step % 2 == 0:
                y = F.gemm(x, wview, b_ready=handle)                      # x @ W^T, K-major B: waits per tile
                ref = x.float() @ ref_w.float().t()
            else:
                y = F.gemm(dyv, wview, b_mn=True, b_ready=handle)         # dy @ W, MN-major B: waits once
                ref = dyv.float() @ ref_w.float()
            torch.cuda.synchronize()
            err = (y.float() - ref).abs().max().item()
            assert err <= 2e-2 * ref.abs().max().item() + 1e-3, f"flag-polling GEMM mismatch at step {step}: {err}"
            dist.barrier()
        # ---- reduce-scatter with fp32 sum, scale, norm and overflow flag.  The pull transport reads the peers'
        # buffers in place, so the gradients then live in symmetric memory.
        gsym = comm.alloc_symmetric(numel, torch.float16) if comm.pulls_gradients else None
        for step in range(3):
            g = torch.Generator(device=dev).manual_seed(7 + 10 * step + rank)
            grad = torch.randn(numel, device=dev, dtype=torch.float16, generator=g)
            if gsym is not None:
                grad = gsym.copy_(grad)
            allg = [torch.empty_like(grad) for _ in range(world)]
            dist.all_gather(allg, grad)
            S = numel // world
            ref = sum(t[rank * S:(rank + 1) * S].float() for t in allg) * 0.5
            shard = torch.empty(S, device=dev, dtype=torch.float16)
            comm.grad_sumsq.zero_()
            comm.overflow.zero_()
            comm.reduce_scatter(shard, grad, key=full, scale=0.5, accumulate_norm=True,
                                stream=torch.cuda.Stream() if step == 2 else None)
            torch.cuda.synchronize()
            assert torch.allclose(shard.float(), ref, rtol=2e-3, atol=2e-3), "reduce_scatter mismatch"
            assert abs(comm.grad_sumsq.item() - ref.pow(2).sum().item()) <= 2e-3 * ref.pow(2).sum().item()
            assert comm.overflow.item() == 0
            dist.barrier()
        grad = torch.full((numel,), float("inf") if rank == 0 else 1.0, device=dev, dtype=torch.float16)
        if gsym is not None:
            grad = gsym.copy_(grad)
        shard = torch.empty(numel // world, device=dev, dtype=torch.float16)
        comm.reduce_scatter(shard, grad, key=full, scale=1.0, accumulate_norm=True)
        torch.cuda.synchronize()
        assert comm.overflow.item() == 1
        dist.barrier()
        # ---- small all-reduce: peer-slot kernel, and the in-switch kernel when a multicast mapping exists
        for dtype in (torch.float16, torch.bfloat16, torch.float32):
            for n in (8, 4096, 65536):
                for use_mc in ([False, True] if comm.heap.multicast_ptr else [False]):
                    for rep in range(3):
                        x = (torch.arange(n, device=dev, dtype=torch.float32) % 7 + rank + rep).to(dtype)
                        ref = x.clone()
                        dist.all_reduce(ref)
                        y = x.clone()
                        comm.all_reduce(y, use_multicast=use_mc)
                        torch.cuda.synchronize()
                        assert torch.allclose(y.float(), ref.float(), rtol=1e-2, atol=1e-2), (dtype, n, use_mc)
        assert _lib.check_status(dev) == 0
        results[rank] = dict(provider=comm.heap.provider, multicast=bool(comm.heap.multicast_ptr),
                             fallback=comm.heap.fallback_reason, all_gather=comm.ag_transport,
                             reduce_scatter=comm.rs_transport)
        dist.barrier()
        comm.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("provider,transport", [("ipc", "sm"), ("auto", "sm"), ("auto", "ce"), ("ipc", "ce"),
                                                ("auto", "mm"), ("ipc", "mm")])
def test_peer_collectives(provider, transport):
    """``mm``: all-gather by multimem.st and reduce-scatter as an owner-side multimem.ld_reduce pull where the heap
    has a multicast mapping; without one (the ``ipc`` mapping) the all-gather falls back to peer DMA and the pull
    reads the peers with plain loads."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), provider, transport, results), nprocs=world, join=True)
        assert len(results) == world
        print("symmetric memory:", dict(results[0]))


def _tp_worker(rank, world, port, results):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from metaseq_b200.ops import _lib
        from metaseq_b200.parallel.symm import TPComm

        M, N, K = 2048, 1024, 512  # K is this rank's slice of the contraction dimension
        tp = TPComm(dist.group.WORLD, dev, max_rows=M, max_cols=N)
        bias = torch.randn(N, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(3))
        resid = torch.randn(M, N, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(4))
        for step in range(4):
            g = torch.Generator(device=dev).manual_seed(50 + 10 * step + rank)
            a = torch.randn(M, K, device=dev, dtype=torch.float16, generator=g)
            w = torch.randn(N, K, device=dev, dtype=torch.float16, generator=g) * 0.05
            ref = a.float() @ w.float().t()
            dist.all_reduce(ref)
            ref = ref + bias.float() + resid.float()
            out = tp.gemm_all_reduce(a, w, bias, resid)
            torch.cuda.synchronize()
            tol = 2e-2 * ref.abs().max().item()
            assert (out.float() - ref).abs().max().item() <= tol, f"gemm_all_reduce mismatch at step {step}"
            rows = M // world
            shard = tp.gemm_reduce_scatter(a, w, bias, resid[rank * rows:(rank + 1) * rows])
            torch.cuda.synchronize()
            assert (shard.float() - ref[rank * rows:(rank + 1) * rows]).abs().max().item() <= tol, "gemm_reduce_scatter mismatch"
            # data-gradient form: dy @ W with W stored [K, N]
            wt = w.t().contiguous()
            out2 = tp.gemm_all_reduce(a, wt, None, None, b_mn=True)
            ref2 = a.float() @ wt.float()
            dist.all_reduce(ref2)
            torch.cuda.synchronize()
            assert (out2.float() - ref2).abs().max().item() <= 2e-2 * ref2.abs().max().item()
        # sequence-parallel all-gather consumed by a GEMM that polls the rows' arrival flags
        from metaseq_b200.ops import functional as F

        calls_before = tp.fused_calls
        for step in range(4):
            g = torch.Generator(device=dev).manual_seed(900 + 10 * step + rank)
            xs = torch.randn(M // world, K, device=dev, dtype=torch.float16, generator=g)
            w = torch.randn(N, K, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(step)) * 0.05
            ref_x = torch.empty(M, K, device=dev, dtype=torch.float16)
            dist.all_gather_into_tensor(ref_x, xs)
            torch.cuda.synchronize()
            dist.barrier()
            full = tp.all_gather_rows(xs)
            if step % 2 == 0:
                y = F.gemm(full, w, bias=bias)                     # [M, K] x [N, K]^T, A polled per tile
                ref = ref_x.float() @ w.float().t() + bias.float()
            else:
                dyv = torch.randn(M, N, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(77))
                y = F.gemm(dyv, full, a_mn=True, b_mn=True)          # weight-gradient form: gathered rows as B
                ref = dyv.float().t() @ ref_x.float()
            torch.cuda.synchronize()
            assert torch.equal(full, ref_x), "gathered rows differ"
            assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3, f"SP gemm mismatch {step}"
            dist.barrier()
        assert tp.fused_calls == calls_before + 4
        assert tp.fused_calls == 16 and tp.fallback_calls == 0
        # vocabulary-parallel cross entropy: kernels + one small all-reduce against full-vocabulary PyTorch
        from metaseq_b200.parallel import mpu, symm
        from metaseq_b200.parallel.cross_entropy import vocab_parallel_cross_entropy

        mpu.initialize_model_parallel(world)
        symm.set_comm_backend("fused")
        Vl, R = 1024, 600
        gen = torch.Generator(device=dev).manual_seed(4242)
        full_logits = torch.randn(R, Vl * world, device=dev, dtype=torch.float16, generator=gen) * 3
        tgt = torch.randint(0, Vl * world, (R,), device=dev, generator=gen)
        tgt[::7] = 1  # padding rows
        local = full_logits[:, rank * Vl:(rank + 1) * Vl].contiguous().requires_grad_(True)
        per_tok = vocab_parallel_cross_entropy(local, tgt, ignore_index=1)
        (per_tok.sum() * 2.0).backward()
        ref_in = full_logits.float().requires_grad_(True)
        ref = torch.nn.functional.cross_entropy(ref_in, tgt, ignore_index=1, reduction="none")
        (ref.sum() * 2.0).backward()
        torch.cuda.synchronize()
        assert torch.allclose(per_tok, ref, rtol=2e-3, atol=2e-3)
        assert torch.allclose(local.grad.float(), ref_in.grad[:, rank * Vl:(rank + 1) * Vl], rtol=2e-2, atol=2e-3)
        assert _lib.check_status(dev) == 0
        results[rank] = True
        dist.barrier()
        tp.close()
    finally:
        dist.destroy_process_group()


def test_gemm_fused_with_tensor_parallel_reduction():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_tp_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert len(results) == world


def _decode_worker(rank, world, port, results):
    """Few-row GEMM fused with the sum over ranks (eager and replayed from a CUDA graph), then the graphed decode
    step of a tensor-parallel model against the module path."""
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from metaseq_b200 import options, tasks
        from metaseq_b200.dataclass.utils import convert_namespace_to_config
        from metaseq_b200.models.decode_step import GraphedDecodeStep
        from metaseq_b200.ops import _lib
        from metaseq_b200.ops import functional as F
        from metaseq_b200.parallel import mpu
        from metaseq_b200.parallel.symm import DecodeReduce

        dev = torch.device("cuda", rank)
        mpu.initialize_model_parallel(world)
        mpu.model_parallel_cuda_manual_seed(7)
        # ---- kernel level
        N, M = 1024, 24
        red = DecodeReduce(dist.group.WORLD, dev, 64, N, torch.float16)
        lib = _lib.kernels()
        split = min(lib.msq_gemm_skinny_split(N, 512), lib.msq_gemm_skinny_split(N, 2048))
        bias = torch.randn(N, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(1))
        res = torch.randn(M, N, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(2))

        def reference(x, w, use_res):
            part = x.float() @ w.float().t()
            part = part.half().float()  # each rank contributes its rounded partial sum
            dist.all_reduce(part)
            return part + bias.float() + (res.float() if use_res else 0.0)

        for step in range(6):
            K = 512 if step % 2 == 0 else 2048
            g = torch.Generator(device=dev).manual_seed(50 + 10 * step + rank)
            x = torch.randn(M, K, device=dev, dtype=torch.float16, generator=g)
            w = torch.randn(N, K, device=dev, dtype=torch.float16, generator=g) * (K ** -0.5)
            y = red.gemm_all_reduce(x, w, bias=bias, residual=res if step % 3 else None, split=split)
            ref = reference(x, w, bool(step % 3))
            torch.cuda.synchronize()
            assert (y.float() - ref).abs().max().item() <= 2e-2, f"fused GEMM + all-reduce mismatch at call {step}"
        # replayed from a graph: four products per replay, inputs refreshed in place between replays
        xs = [torch.zeros(M, K, device=dev, dtype=torch.float16) for K in (512, 2048, 512, 2048)]
        ws = [torch.randn(N, K, device=dev, dtype=torch.float16, generator=torch.Generator(device=dev).manual_seed(9 + i + 4 * rank))
              * (K ** -0.5) for i, K in enumerate((512, 2048, 512, 2048))]

        def four():
            return [red.gemm_all_reduce(x, w, bias=bias, residual=res, split=split) for x, w in zip(xs, ws)]

        with F.dependent_launch():
            four()
            torch.cuda.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                outs = four()
        for it in range(4):
            for i, x in enumerate(xs):
                x.copy_(torch.randn(x.shape, device=dev, dtype=torch.float16,
                                    generator=torch.Generator(device=dev).manual_seed(1000 + 100 * it + 10 * i + rank)))
            graph.replay()
            torch.cuda.synchronize()
            for x, w, y in zip(xs, ws, outs):
                ref = reference(x, w, True)
                assert (y.float() - ref).abs().max().item() <= 2e-2, f"graph replay {it}: mismatch"
        assert _lib.check_status(dev) == 0
        # ---- model level
        parser = options.get_training_parser()
        ns = options.parse_args_and_arch(parser, input_args=[
            "--task", "dummy_lm", "--dict-size", "2040", "--tokens-per-sample", "128", "--batch-size", "1",
            "--arch", "transformer_lm_megatron", "--decoder-layers", "3", "--decoder-embed-dim", "512",
            "--decoder-ffn-embed-dim", "2048", "--decoder-attention-heads", "8", "--decoder-learned-pos",
            "--activation-fn", "relu", "--share-decoder-input-output-embed", "--no-scale-embedding", "--dropout", "0.0",
            "--attention-dropout", "0.0", "--criterion", "vocab_parallel_cross_entropy", "--optimizer", "adam",
            "--lr", "1e-3", "--memory-efficient-fp16", "--tensor-parallel-init-model-on-gpu",
            "--distributed-world-size", str(world), "--model-parallel-size", str(world)])
        cfg = convert_namespace_to_config(ns)
        task = tasks.setup_task(cfg.task)
        torch.manual_seed(3)
        model = task.build_model(cfg.model).half().cuda().eval()
        model.make_generation_fast_()
        dec = model.decoder
        assert GraphedDecodeStep.supported(dec, 3)
        tokens = torch.randint(4, 2000, (3, 40), device=dev, generator=torch.Generator(device=dev).manual_seed(11))
        with torch.no_grad():
            full, _ = model(tokens)  # gathered logits [3, 40, V]
            runner = GraphedDecodeStep.for_decoder(dec, 3, 64)
            model(tokens[:, :24], incremental_state=runner.new_state())
            runner.begin(tokens[:, :24])
            for t in range(24, 39):
                logits = runner.step(tokens[:, t])
                assert logits.shape == full[:, t].shape
                torch.testing.assert_close(logits.float(), full[:, t].float(), rtol=5e-2, atol=5e-2)
        assert runner.reduce is not None and runner.reduce.calls > 0
        assert _lib.check_status(dev) == 0
        # ---- the small exchange kernel on its own: sum of 16-bit rows and all-gather of records, eager and replayed
        from metaseq_b200.parallel.symm import WordsExchange

        ex = WordsExchange(dist.group.WORLD, dev, 4096)
        for it in range(3):
            g = torch.Generator(device=dev).manual_seed(300 + 10 * it + rank)
            x = torch.randn(5, 256, device=dev, dtype=torch.float16, generator=g)
            ref = x.float()
            dist.all_reduce(ref)
            torch.testing.assert_close(ex.sum(x).float(), ref, rtol=2e-3, atol=2e-3)
            rec = torch.randn(7, 4, device=dev, generator=g)
            every = ex.gather(rec)
            refs = [torch.empty_like(rec) for _ in range(world)]
            dist.all_gather(refs, rec)
            assert torch.equal(every, torch.stack(refs))
        xg = torch.zeros(6, 128, device=dev, dtype=torch.float16)
        ex.sum(xg)
        torch.cuda.synchronize()
        dist.barrier()
        gx = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gx):
            yg = ex.sum(xg)
        for it in range(4):
            xg.copy_(torch.randn(6, 128, device=dev, generator=torch.Generator(device=dev).manual_seed(40 + it + 7 * rank)))
            gx.replay()
            ref = xg.float()
            dist.all_reduce(ref)
            torch.testing.assert_close(yg.float(), ref, rtol=2e-3, atol=2e-3)
        # ---- greedy generation: tokens picked from the logit shards equal those picked from gathered logits
        from metaseq_b200.sequence_generator import SequenceGenerator

        prompts = tokens[:, :16].contiguous()
        outs = {}
        for shard_picks in (True, False):
            sg = SequenceGenerator([model], task.target_dictionary, beam_size=1, max_len_b=40, min_len=30, temperature=1.0,
                                   topp=-1.0, decode_graph=True)
            sg.shard_picks = shard_picks
            with torch.no_grad():
                outs[shard_picks] = sg.generate([model], {"net_input": {"src_tokens": prompts}})
        assert torch.equal(outs[True]["tokens"], outs[False]["tokens"])
        torch.testing.assert_close(outs[True]["scores"], outs[False]["scores"], rtol=1e-3, atol=2e-3)
        assert _lib.check_status(dev) == 0
        results[rank] = True
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_decode_gemm_fused_with_all_reduce_and_graphed_tensor_parallel_step(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs at least {world} GPUs")
    import torch.multiprocessing as mp

    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_decode_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert all(results.get(r) for r in range(world))
