"""Tensor-parallel training on two GPUs: the fused (peer-memory) and the NCCL communication backends must
produce the same losses."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(backend, tmp_path, extra=()):
    save = tmp_path / f"ckpt_{backend}"
    cmd = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
        "--master-port", str(_free_port()), "-m", "metaseq_b200.cli.train",
        "--task", "dummy_lm", "--dict-size", "1020", "--tokens-per-sample", "256", "--batch-size", "4",
        "--arch", "transformer_lm_megatron", "--decoder-layers", "2", "--decoder-embed-dim", "256",
        "--decoder-ffn-embed-dim", "1024", "--decoder-attention-heads", "4", "--decoder-learned-pos", "--activation-fn", "relu",
        "--share-decoder-input-output-embed", "--no-scale-embedding", "--dropout", "0.0", "--attention-dropout", "0.0",
        "--criterion", "vocab_parallel_cross_entropy", "--optimizer", "adam", "--adam-betas", "(0.9, 0.95)",
        "--lr", "1e-3", "--lr-scheduler", "polynomial_decay", "--warmup-updates", "2", "--total-num-update", "100",
        "--clip-norm", "1.0", "--memory-efficient-fp16", "--fp16-init-scale", "4", "--ddp-backend", "fully_sharded",
        "--use-sharded-state", "--no-reshard-after-forward", "--tensor-parallel-init-model-on-gpu",
        "--distributed-world-size", "2", "--model-parallel-size", "2", "--max-update", "6", "--log-format", "json",
        "--log-interval", "1", "--save-dir", str(save), "--disable-validation", "--save-interval-epochs", "0", "--save-interval-updates", "0", "--seed", "3",
        "--comm-backend", backend, *extra,
    ]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    losses = []
    for line in out.stdout.splitlines():
        i = line.find('{"epoch"')
        if i >= 0 and '"loss"' in line:
            rec = json.loads(line[i:])
            if "num_updates" in rec and "train_loss" not in rec:
                losses.append(float(rec["loss"]))
    return losses, out.stdout


@pytest.mark.parametrize("sp", [False, True])
def test_tensor_parallel_fused_matches_nccl(tmp_path, sp):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    extra = ("--sequence-parallel",) if sp else ()
    fused, log = _run("fused", tmp_path, extra)
    nccl, _ = _run("nccl", tmp_path, extra)
    assert len(fused) >= 5 and len(fused) == len(nccl), log[-2000:]
    assert "TPComm: fused GEMM -> " + ("reduce-scatter" if sp else "all-reduce") + " active" in log, log[-3000:]
    if sp:
        assert "TPComm: fused all-gather -> GEMM active" in log
    for a, b in zip(fused, nccl):
        assert abs(a - b) <= 2e-2 * max(1.0, abs(b)), (fused, nccl)
    assert fused[-1] < fused[0]


def _run_fsdp(save, max_update, extra=(), env=None, backend="fused"):
    cmd = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
        "--master-port", str(_free_port()), "-m", "metaseq_b200.cli.train",
        "--task", "dummy_lm", "--dict-size", "1020", "--tokens-per-sample", "256", "--batch-size", "4",
        "--arch", "transformer_lm_megatron", "--decoder-layers", "2", "--decoder-embed-dim", "256",
        "--decoder-ffn-embed-dim", "1024", "--decoder-attention-heads", "4", "--decoder-learned-pos", "--activation-fn", "relu",
        "--share-decoder-input-output-embed", "--no-scale-embedding", "--dropout", "0.1", "--attention-dropout", "0.0",
        "--criterion", "vocab_parallel_cross_entropy", "--optimizer", "adam", "--adam-betas", "(0.9, 0.95)",
        "--lr", "1e-3", "--lr-scheduler", "polynomial_decay", "--warmup-updates", "2", "--total-num-update", "100",
        "--clip-norm", "1.0", "--memory-efficient-fp16", "--fp16-init-scale", "4", "--ddp-backend", "fully_sharded",
        "--use-sharded-state", "--no-reshard-after-forward", "--tensor-parallel-init-model-on-gpu",
        "--distributed-world-size", "2", "--max-update", str(max_update), "--log-format", "json", "--log-interval", "1",
        "--save-dir", str(save), "--disable-validation", "--save-interval-epochs", "0", "--save-interval-updates", "3",
        "--seed", "3", "--comm-backend", backend, *extra,
    ]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, OMP_NUM_THREADS="1", **(env or {})))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    losses = {}
    for line in out.stdout.splitlines():
        i = line.find('{"epoch"')
        if i >= 0 and '"loss"' in line:
            rec = json.loads(line[i:])
            if "num_updates" in rec and "train_loss" not in rec:
                losses[int(rec["num_updates"])] = float(rec["loss"])
    return losses


def test_sharded_checkpoint_resume_with_peer_memory_collectives(tmp_path):
    """Two data-parallel GPUs with the peer-memory all-gather / reduce-scatter: a run resumed from the sharded
    checkpoint of update 3 continues like the uninterrupted run (weights gathered again from the restored shards,
    optimizer state, loss scale, dropout seeds)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import shutil

    straight = _run_fsdp(tmp_path / "a", 6)
    assert sorted(straight) == [1, 2, 3, 4, 5, 6]
    resumed_dir = tmp_path / "b"
    resumed_dir.mkdir()
    for name in os.listdir(tmp_path / "a"):
        if name.startswith("checkpoint_3"):
            shutil.copy(tmp_path / "a" / name, resumed_dir / name.replace("checkpoint_3", "checkpoint_last"))
    assert len(os.listdir(resumed_dir)) == 2, os.listdir(tmp_path / "a")
    resumed = _run_fsdp(resumed_dir, 6)
    assert sorted(resumed) == [4, 5, 6], resumed
    for n in (4, 5, 6):
        assert resumed[n] == pytest.approx(straight[n], abs=2e-2), (n, resumed, straight)


@pytest.mark.parametrize("transport", ["mm", "sm"])
def test_fsdp_collectives_through_the_switch_match_nccl(tmp_path, transport):
    """Two data-parallel GPUs, gradient accumulation over two micro-batches: the all-gather by multimem.st with the
    owner-side multimem.ld_reduce reduce-scatter (``mm``) and the store kernels (``sm``) give the losses of the NCCL run."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    extra = ("--update-freq", "2")
    ours = _run_fsdp(tmp_path / transport, 5, extra, env={"MSQ_COMM_TRANSPORT": transport})
    nccl = _run_fsdp(tmp_path / "nccl", 5, extra, backend="nccl")
    assert sorted(ours) == sorted(nccl) == [1, 2, 3, 4, 5]
    for n in nccl:
        assert ours[n] == pytest.approx(nccl[n], abs=2e-2), (n, ours, nccl)
    assert ours[5] < ours[1]
