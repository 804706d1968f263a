"""End-to-end training on CPU with gloo ranks, through the real command line: data-parallel FSDP against one rank,
tensor parallelism against one rank, checkpoint names, resume determinism, restoring on a different number of
ranks, and the offline reshard / consolidate tools."""
import glob
import json
import os
import subprocess
import sys

import pytest
import torch

COMMON = [
    "--task", "dummy_lm", "--dict-size", "508", "--tokens-per-sample", "32", "--batch-size", "2",
    "--arch", "transformer_lm_megatron", "--decoder-layers", "2", "--decoder-embed-dim", "64",
    "--decoder-ffn-embed-dim", "256", "--decoder-attention-heads", "2", "--decoder-learned-pos",
    "--share-decoder-input-output-embed", "--activation-fn", "relu", "--dropout", "0.0", "--attention-dropout", "0.0",
    "--criterion", "vocab_parallel_cross_entropy", "--optimizer", "adam", "--lr", "1e-3", "--lr-scheduler",
    "polynomial_decay", "--total-num-update", "100", "--warmup-updates", "2", "--clip-norm", "1.0",
    "--ddp-backend", "fully_sharded", "--use-sharded-state", "--log-format", "json", "--log-interval", "1",
    "--disable-validation", "--cpu", "--seed", "5",
]


def run_train(save_dir, world, max_update, extra=()):
    cmd = [sys.executable, "-m", "metaseq_b200.cli.train", *COMMON, "--distributed-world-size", str(world),
           "--max-update", str(max_update), "--save-dir", str(save_dir), *extra]
    env = dict(os.environ, OMP_NUM_THREADS="2", MASTER_ADDR="127.0.0.1")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    losses = {}
    for line in out.stdout.splitlines():
        i = line.find('{"epoch"')
        if i >= 0:
            rec = json.loads(line[i:])
            if "num_updates" in rec and "loss" in rec and "train_loss" not in rec:
                losses[int(rec["num_updates"])] = (float(rec["loss"]), float(rec.get("gnorm", 0)))
    return losses, out.stdout


@pytest.fixture(scope="module")
def runs(tmp_path_factory):
    root = tmp_path_factory.mktemp("train")
    r = {}
    r["dp1"], _ = run_train(root / "dp1", 1, 6)
    r["dp2"], _ = run_train(root / "dp2", 2, 4, ["--save-interval-updates", "3"])
    r["root"] = root
    return r


def test_two_data_parallel_ranks_match_one_rank(runs):
    # every rank draws the same synthetic batch, so averaging over two ranks reproduces the single-rank run
    for step in range(1, 5):
        assert runs["dp2"][step][0] == pytest.approx(runs["dp1"][step][0], abs=2e-3)
        assert runs["dp2"][step][1] == pytest.approx(runs["dp1"][step][1], rel=2e-2)
    assert runs["dp1"][6][0] < runs["dp1"][1][0]


def test_checkpoint_files_follow_the_sharded_naming_scheme(runs):
    names = sorted(os.path.basename(p) for p in glob.glob(str(runs["root"] / "dp2" / "*.pt")))
    assert names == ["checkpoint_3-model_part-0-shard0.pt", "checkpoint_3-model_part-0-shard1.pt",
                     "checkpoint_last-model_part-0-shard0.pt", "checkpoint_last-model_part-0-shard1.pt"]
    state = torch.load(runs["root"] / "dp2" / "checkpoint_last-model_part-0-shard1.pt", map_location="cpu",
                       weights_only=False)
    assert "shard_metadata" in state and any(k.endswith("flat_param_0") for k in state["model"])
    assert state["optimizer_history"][-1]["num_updates"] == 4
    assert "last_optimizer_state" in state and "extra_state" in state


def test_resume_continues_the_same_trajectory(runs):
    resumed, log = run_train(runs["root"] / "dp2", 2, 6)
    assert "Loaded checkpoint" in log or "loaded checkpoint" in log.lower()
    assert min(resumed) == 5  # picks up after update 4
    for step in (5, 6):
        assert resumed[step][0] == pytest.approx(runs["dp1"][step][0], abs=3e-3)


def test_restore_on_fewer_ranks(runs, tmp_path):
    # two shard files restored by a single rank (a data-parallel resize)
    src = runs["root"] / "dp2" / "checkpoint_3-model_part-0-shard0.pt"
    resized, log = run_train(tmp_path / "resized", 1, 5, ["--restore-file", str(src).replace("-shard0", "")])
    assert min(resized) == 4
    assert resized[4][0] == pytest.approx(runs["dp1"][4][0], abs=3e-3)
    assert resized[5][0] == pytest.approx(runs["dp1"][5][0], abs=3e-3)


def test_tensor_parallel_matches_single_rank(tmp_path, runs):
    tp2, _ = run_train(tmp_path / "tp2", 2, 3, ["--model-parallel-size", "2"])
    for step in range(1, 4):
        assert tp2[step][0] == pytest.approx(runs["dp1"][step][0], abs=5e-3)
    names = sorted(os.path.basename(p) for p in glob.glob(str(tmp_path / "tp2" / "checkpoint_last*")))
    assert names == ["checkpoint_last-model_part-0-shard0.pt", "checkpoint_last-model_part-1-shard0.pt"]


def test_reshard_and_consolidate_tools_roundtrip(runs, tmp_path):
    from metaseq_b200.checkpoint import consolidate_fsdp_shards, reshard_fsdp

    src = str(runs["root"] / "dp2" / "checkpoint_last-model_part-0-shard*.pt")
    one = str(tmp_path / "one" / "reshard-model_part-0-shard{i}.pt")
    reshard_fsdp.reshard_fsdp_checkpoints(src, one, num_output_shards=1)
    two = str(tmp_path / "two" / "reshard-model_part-0-shard{i}.pt")
    reshard_fsdp.reshard_fsdp_checkpoints(one.replace("{i}", "*"), two, num_output_shards=2)
    a = [torch.load(p, map_location="cpu", weights_only=False) for p in sorted(glob.glob(src))]
    b = [torch.load(p, map_location="cpu", weights_only=False) for p in sorted(glob.glob(two.replace("{i}", "*")))]
    assert len(b) == 2
    for sa, sb in zip(a, b):
        for k, v in sa["model"].items():
            if torch.is_tensor(v):
                assert torch.equal(v, sb["model"][k]), k
    unflat = reshard_fsdp.reshard_fsdp_checkpoints(src, str(tmp_path / "unflat" / "model-shard{i}.pt"),
                                                   num_output_shards=1, unflatten_weights=True)
    full = torch.load(glob.glob(str(tmp_path / "unflat" / "*.pt"))[0], map_location="cpu", weights_only=False)["model"]
    assert "decoder.layers.0.self_attn.qkv_proj.weight" in full
    assert full["decoder.layers.0.self_attn.qkv_proj.weight"].shape == (192, 64)
    assert not any("flat_param" in k for k in full)
