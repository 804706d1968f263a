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


def test_gradient_accumulation_over_two_ranks_matches_one_rank(tmp_path):
    """``--update-freq 2``: each micro-batch's reduced gradient is added once.  Every rank draws the same synthetic
    batches, so loss and gradient norm agree between one rank and two."""
    one, _ = run_train(tmp_path / "one", 1, 3, ["--update-freq", "2"])
    two, _ = run_train(tmp_path / "two", 2, 3, ["--update-freq", "2"])
    for step in range(1, 4):
        assert two[step][0] == pytest.approx(one[step][0], abs=2e-3)
        assert two[step][1] == pytest.approx(one[step][1], rel=2e-2)


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


def test_tensor_parallel_tool_chain_rebuilds_a_single_rank_model(tmp_path):
    """Two tensor-parallel ranks train and save; the offline tools unflatten each part, merge the parts into one,
    write the singleton file, re-split it, and the FasterTransformer converter reads it.  The merged weights,
    loaded into a single-rank model, reproduce the next training loss of the two-rank run."""
    from metaseq_b200.checkpoint import convert_metaseq_ft, convert_to_singleton, reshard_consolidated, reshard_fsdp, reshard_mp

    tp2, _ = run_train(tmp_path / "tp2", 2, 3, ["--model-parallel-size", "2", "--save-interval-updates", "3"])
    ckpt_dir = tmp_path / "tp2"
    for part in (0, 1):
        reshard_fsdp.reshard_fsdp_checkpoints(str(ckpt_dir / f"checkpoint_last-model_part-{part}-shard*.pt"),
                                              str(tmp_path / "unflat" / f"reshard-model_part-{part}-shard{{i}}.pt"),
                                              num_output_shards=1, unflatten_weights=True)
        os.rename(tmp_path / "unflat" / f"reshard-model_part-{part}-shard0.pt", tmp_path / "unflat" / f"reshard-model_part-{part}.pt")
    parts = [torch.load(tmp_path / "unflat" / f"reshard-model_part-{p}.pt", map_location="cpu", weights_only=False)["model"]
             for p in (0, 1)]
    one = reshard_mp.reshard_mp(str(tmp_path / "unflat" / "reshard-model_part-*.pt"), str(tmp_path / "mp1" / "reshard-model_part-{i}.pt"), 1)
    merged = torch.load(one[0], map_location="cpu", weights_only=False)["model"]
    D = 64
    qkv = "decoder.layers.0.self_attn.qkv_proj.weight"
    assert merged[qkv].shape == (3 * D, D)
    for j in range(3):  # k | v | q blocks: each is the concatenation of the two ranks' halves of that block
        want = torch.cat([p[qkv][j * D // 2:(j + 1) * D // 2] for p in parts])
        assert torch.equal(merged[qkv][j * D:(j + 1) * D], want)
    fc2 = "decoder.layers.1.fc2.weight"
    assert torch.equal(merged[fc2], torch.cat([p[fc2] for p in parts], dim=1))
    assert torch.equal(merged["decoder.layers.0.self_attn_layer_norm.weight"], parts[0]["decoder.layers.0.self_attn_layer_norm.weight"])
    # singleton file from the two parts equals the one-part reshard
    single = convert_to_singleton.convert_to_singleton(str(tmp_path / "unflat"))
    restored = torch.load(single, map_location="cpu", weights_only=False)["model"]
    assert all(torch.equal(restored[k], merged[k]) for k in merged if torch.is_tensor(merged[k]))
    # and splits back into the original two parts
    back = reshard_mp.reshard_mp(one[0], str(tmp_path / "mp2" / "reshard-model_part-{i}.pt"), 2)
    for p, path in zip(parts, back):
        again = torch.load(path, map_location="cpu", weights_only=False)["model"]
        assert all(torch.equal(again[k], p[k]) for k in p if torch.is_tensor(p[k]))
    # the merged weights in a one-rank model give the loss the two-rank run reported next
    from metaseq_b200 import options, tasks
    from metaseq_b200.dataclass.utils import convert_namespace_to_config

    argv = [a for a in COMMON if a not in ("--ddp-backend", "fully_sharded", "--use-sharded-state")] + \
        ["--distributed-world-size", "1", "--criterion", "cross_entropy"]
    cfg = convert_namespace_to_config(options.parse_args_and_arch(options.get_training_parser(), input_args=argv))
    task = tasks.setup_task(cfg.task)
    model = task.build_model(cfg.model).eval()
    missing, unexpected = model.load_state_dict({k: v for k, v in merged.items() if torch.is_tensor(v)}, strict=False)
    assert not [m for m in missing if "version" not in m] and not [u for u in unexpected if "version" not in u], (missing, unexpected)
    task.load_dataset("train")
    batch = task.dataset("train").collater([0, 1])
    with torch.no_grad():
        logits, _ = model(**batch["net_input"])
        nll = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(), batch["target"].view(-1),
                                                reduction="mean")
    four, _ = run_train(tmp_path / "tp2", 2, 4, ["--model-parallel-size", "2", "--save-interval-updates", "3"])
    assert float(nll) / 0.6931471805599453 == pytest.approx(four[4][0], abs=2e-2)  # logged in bits per token
    # sharded again for FSDP, and exported for FasterTransformer
    shards = reshard_consolidated.reshard_consolidated(single, str(tmp_path / "fsdp" / "reshard-model_part-0-shard{i}.pt"), 2)
    assert len(shards) == 2
    convert_metaseq_ft.convert_metaseq_ft(single, str(tmp_path / "ft" / "part-{i}.pt"), dtype="fp32")
    ft = torch.load(tmp_path / "ft" / "part-0.pt", map_location="cpu", weights_only=False)["weights"]
    layers = 2
    assert len(ft) == 12 * layers + 5
    ft_qkv = ft[2 * layers]  # third per-layer slot, layer 0: the fused projection reordered from (k, v, q) to (q, k, v)
    k, v, q = merged[qkv][:D], merged[qkv][D:2 * D], merged[qkv][2 * D:]
    assert ft_qkv.numel() == 3 * D * D
    flat = ft_qkv.reshape(-1)
    assert any(torch.equal(flat, c.reshape(-1)) for c in (torch.cat([q, k, v]).t().contiguous(), torch.cat([q, k, v]),
                                                          torch.stack([q, k, v], 0).permute(2, 0, 1).contiguous()))
    assert ft[12 * layers + 2].shape[0] == merged["decoder.embed_positions.weight"].shape[0] - 2  # first two rows dropped


def test_ddp_backend_matches_fully_sharded(tmp_path, runs):
    """``--ddp-backend pytorch_ddp`` (replicated parameters, bucketed gradient all-reduce) follows the same
    trajectory as the fully sharded run on two ranks and writes one consolidated file per model part."""
    args = [a for a in COMMON if a not in ("--ddp-backend", "fully_sharded", "--use-sharded-state")]
    cmd = [sys.executable, "-m", "metaseq_b200.cli.train", *args, "--ddp-backend", "pytorch_ddp",
           "--distributed-world-size", "2", "--max-update", "4", "--save-dir", str(tmp_path / "ddp"),
           "--save-interval-updates", "4"]
    env = dict(os.environ, OMP_NUM_THREADS="2", MASTER_ADDR="127.0.0.1")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    losses = {}
    for line in out.stdout.splitlines():
        i = line.find('{"epoch"')
        if i >= 0:
            rec = json.loads(line[i:])
            if "num_updates" in rec and "loss" in rec and "train_loss" not in rec:
                losses[int(rec["num_updates"])] = float(rec["loss"])
    assert sorted(losses) == [1, 2, 3, 4]
    for step in range(1, 5):
        assert losses[step] == pytest.approx(runs["dp2"][step][0], abs=5e-3)
    names = sorted(os.path.basename(p) for p in glob.glob(str(tmp_path / "ddp" / "checkpoint_last*")))
    assert names == ["checkpoint_last-model_part-0.pt"]


def test_restore_on_more_ranks(runs, tmp_path):
    """Two shard files restored by four ranks (the reference trains on 2 GPUs and restores on 4:
    gpu_tests/test_checkpoint_loading_on_more_gpus.py): the run continues and writes four shard files."""
    src = runs["root"] / "dp2" / "checkpoint_3-model_part-0-shard0.pt"
    # four ranks see twice the data per update, so only the first restored update is comparable through its loss on the
    # fixed synthetic batch (every rank gets the same batch): equal to the one-rank run
    resized, log = run_train(tmp_path / "wide", 4, 5, ["--restore-file", str(src).replace("-shard0", ""),
                                                      "--save-interval-updates", "5"])
    assert min(resized) == 4
    assert resized[4][0] == pytest.approx(runs["dp1"][4][0], abs=3e-3)
    names = sorted(os.path.basename(p) for p in glob.glob(str(tmp_path / "wide" / "checkpoint_last*")))
    assert names == [f"checkpoint_last-model_part-0-shard{i}.pt" for i in range(4)]


def test_async_sharded_save_then_reshard_to_fewer_model_parts_and_reload(tmp_path):
    """The checkpoint path of the large tensor-parallel recipe at toy size: four tensor-parallel ranks train and save
    their shards through the asynchronous writer; the offline tools unflatten every part and re-split the model for
    two tensor-parallel ranks; a two-rank run restored from those files computes, on its first update, the loss that
    the four-rank run reports on its next one."""
    from metaseq_b200.checkpoint import reshard_fsdp, reshard_mp

    heads4 = ["--decoder-attention-heads", "4", "--model-parallel-size", "4", "--write-checkpoints-asynchronously",
              "--save-interval-updates", "3"]
    run_train(tmp_path / "tp4", 4, 3, heads4)
    names = sorted(os.path.basename(p) for p in glob.glob(str(tmp_path / "tp4" / "checkpoint_3*")))
    assert names == [f"checkpoint_3-model_part-{i}-shard0.pt" for i in range(4)]  # all written, none left as .tmp
    for part in range(4):
        reshard_fsdp.reshard_fsdp_checkpoints(str(tmp_path / "tp4" / f"checkpoint_3-model_part-{part}-shard*.pt"),
                                              str(tmp_path / "unflat" / f"reshard-model_part-{part}-shard{{i}}.pt"),
                                              num_output_shards=1, unflatten_weights=True)
        os.rename(tmp_path / "unflat" / f"reshard-model_part-{part}-shard0.pt",
                  tmp_path / "unflat" / f"reshard-model_part-{part}.pt")
    two = reshard_mp.reshard_mp(str(tmp_path / "unflat" / "reshard-model_part-*.pt"),
                                str(tmp_path / "tp2" / "resharded-model_part-{i}.pt"), 2)
    assert [os.path.basename(p) for p in two] == ["resharded-model_part-0.pt", "resharded-model_part-1.pt"]
    cont, _ = run_train(tmp_path / "tp4", 4, 4, heads4)  # the four-rank run goes on: update 4
    flags = [a for a in COMMON if a != "--use-sharded-state"]
    cmd = [sys.executable, "-m", "metaseq_b200.cli.train", *flags, "--decoder-attention-heads", "4",
           "--model-parallel-size", "2", "--distributed-world-size", "2", "--max-update", "1",
           "--save-dir", str(tmp_path / "tp2run"), "--restore-file", str(tmp_path / "tp2" / "resharded.pt"),
           "--reset-optimizer", "--reset-dataloader", "--reset-meters", "--reset-lr-scheduler",
           "--save-interval-updates", "0", "--save-interval-epochs", "0"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, OMP_NUM_THREADS="2", MASTER_ADDR="127.0.0.1"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    first = None
    for line in out.stdout.splitlines():
        i = line.find('{"epoch"')
        if i >= 0:
            rec = json.loads(line[i:])
            if "num_updates" in rec and "loss" in rec and "train_loss" not in rec:
                first = float(rec["loss"])
                break
    assert first is not None, out.stdout[-2000:]
    assert first == pytest.approx(cont[4][0], abs=5e-3)


def test_sharded_checkpoints_on_a_shared_directory_resume_only_from_a_complete_set(tmp_path):
    """Two data-parallel ranks with sharded state and ``--cloud-upload-path nfs:<dir>``: every rank moves its own
    shard into ``checkpoint_N/``; a restart takes the newest directory that holds one finished file per rank, and an
    incomplete newer directory (a rank died mid-copy) is passed over."""
    shared = tmp_path / "shared"
    shared.mkdir()
    extra = ["--save-interval-updates", "2", "--cloud-upload-path", f"nfs:{shared}"]
    losses, _ = run_train(tmp_path / "a", 2, 4, extra)
    assert sorted(losses) == [1, 2, 3, 4]
    names = sorted(p.name for p in (shared / "checkpoint_4").iterdir())
    assert names == ["checkpoint-model_part-0-shard0.pt", "checkpoint-model_part-0-shard1.pt"], names
    # a newer checkpoint with one part still being copied must not be chosen
    broken = shared / "checkpoint_6"
    broken.mkdir()
    (broken / "checkpoint-model_part-0-shard0.pt").write_bytes(b"partial set")
    (broken / "_checkpoint-model_part-0-shard1.pt").write_bytes(b"in flight")
    resumed, log = run_train(tmp_path / "b", 2, 6, extra)
    assert sorted(resumed) == [5, 6], (sorted(resumed), log[-1500:])
    assert "skipping checkpoint checkpoint_6" in log
