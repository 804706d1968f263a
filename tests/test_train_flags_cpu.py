"""Every training option that changes the numerical path runs a few updates on a CPU without error and with a
finite, falling loss on the fixed synthetic batch."""
import math

import pytest
import torch

from metaseq_b200 import options, tasks
from metaseq_b200.cli.train import build_model_and_criterion
from metaseq_b200.dataclass.utils import convert_namespace_to_config
from metaseq_b200.trainer import Trainer

POLY = ["--lr-scheduler", "polynomial_decay", "--total-num-update", "100", "--warmup-updates", "1"]
VARIANTS = {
    "default": POLY,
    "bf16": POLY + ["--bf16"],
    "fp16_master_weights": POLY + ["--fp16", "--fp16-init-scale", "4"],
    "memory_efficient_fp16": POLY + ["--memory-efficient-fp16", "--fp16-init-scale", "4"],
    "activation_checkpointing": POLY + ["--checkpoint-activations"],
    "seed_per_rank": POLY + ["--seed-per-rank", "--dropout", "0.1"],
    "recompute_first_layer": POLY + ["--recompute-fc1-num-layers", "1"],
    "offloaded_checkpoints": POLY + ["--checkpoint-activations", "--offload-activations"],
    "activation_checkpointing_modular_layer": POLY + ["--checkpoint-activations", "--no-fused-layer", "--dropout", "0.1"],
    "sgd": POLY + ["--optimizer", "sgd", "--momentum", "0.9"],
    "cosine": ["--lr-scheduler", "cosine", "--max-lr", "1e-2", "--lr-period-updates", "10", "--warmup-updates", "1"],
    "inverse_sqrt": ["--lr-scheduler", "inverse_sqrt", "--warmup-init-lr", "1e-4", "--warmup-updates", "1"],
    "modular_layer": POLY + ["--no-fused-layer"],
    "gelu": POLY + ["--activation-fn", "gelu"],
    "alibi": POLY + ["--alibi"],
    "document_separator_attention": POLY + ["--self-attn-doc-sep", "2"],
    "sinusoidal_positions": POLY + ["--decoder-learned-sinusoidal"],
    "vocab_parallel_criterion": POLY + ["--criterion", "vocab_parallel_cross_entropy"],
    "dropout": POLY + ["--dropout", "0.1", "--attention-dropout", "0.1"],
    "fully_sharded": POLY + ["--ddp-backend", "fully_sharded", "--use-sharded-state"],
    "fp16_adam_stats": POLY + ["--memory-efficient-fp16", "--fp16-init-scale", "4", "--fp16-adam-stats"],
    "loss_spike_guard": POLY + ["--ewm-ratio-to-skip-batch", "2.0"],
    "two_layers_per_sharded_unit": POLY + ["--ddp-backend", "fully_sharded", "--checkpoint-activations",
                                           "--fsdp-checkpoint-wrap-layer-frequency", "2"],
}


def _run(save_dir, extra, updates=6):
    argv = ["--task", "dummy_lm", "--dict-size", "124", "--tokens-per-sample", "16", "--batch-size", "2",
            "--arch", "transformer_lm_megatron", "--decoder-layers", "2", "--decoder-embed-dim", "32",
            "--decoder-ffn-embed-dim", "64", "--decoder-attention-heads", "2", "--decoder-learned-pos",
            "--share-decoder-input-output-embed", "--dropout", "0.0", "--attention-dropout", "0.0", "--criterion",
            "cross_entropy", "--optimizer", "adam", "--lr", "1e-2", "--clip-norm", "1.0", "--cpu",
            "--distributed-world-size", "1", "--save-dir", str(save_dir), "--disable-validation", "--log-format", "none",
            *extra]
    cfg = convert_namespace_to_config(options.parse_args_and_arch(options.get_training_parser(), input_args=argv))
    torch.manual_seed(1)
    task = tasks.setup_task(cfg.task)
    model, criterion = build_model_and_criterion(cfg, task)
    tr = Trainer(cfg, task, model, criterion)
    task.load_dataset("train")
    batch = task.dataset("train").collater([0, 1])
    losses = []
    for _ in range(updates):
        log = tr.train_step([batch])
        if log is not None:  # an overflow step of the dynamic loss scaler returns nothing
            losses.append(float(log["loss"]))
    return losses


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_training_option_runs_and_learns(name, tmp_path):
    losses = _run(tmp_path, VARIANTS[name])
    assert len(losses) >= 4 and all(math.isfinite(v) for v in losses), losses
    assert losses[-1] < losses[0], (name, losses)


def test_cpu_offload_keeps_shards_on_the_host_and_trains_like_the_plain_run(tmp_path):
    """``--cpu-offload`` on a CPU-only host moves nothing, so the run must equal the one without the flag; the unit
    still goes through the offload path (separate gathered copy, gradient copied back to the shard's device)."""
    base = _run(tmp_path / "a", POLY + ["--ddp-backend", "fully_sharded"])
    off = _run(tmp_path / "b", POLY + ["--ddp-backend", "fully_sharded", "--cpu-offload"])
    assert off == pytest.approx(base, abs=1e-4)


@pytest.mark.parametrize("flags", [["--fp16", "--fp16-init-scale", "4"], ["--cpu-offload"], []])
def test_two_identical_micro_batches_give_the_update_of_one(tmp_path, flags):
    """Sharded model on one rank, also with fp32 master shards or offloaded shards (where the flat gradient buffer
    is not the parameter's gradient): accumulating two copies of a batch must not count the first one twice."""
    extra = POLY + ["--ddp-backend", "fully_sharded", "--clip-norm", "0.0"] + flags

    def run(copies):
        argv = ["--task", "dummy_lm", "--dict-size", "124", "--tokens-per-sample", "16", "--batch-size", "2",
                "--arch", "transformer_lm_megatron", "--decoder-layers", "2", "--decoder-embed-dim", "32",
                "--decoder-ffn-embed-dim", "64", "--decoder-attention-heads", "2", "--decoder-learned-pos",
                "--share-decoder-input-output-embed", "--dropout", "0.0", "--attention-dropout", "0.0", "--criterion",
                "cross_entropy", "--optimizer", "adam", "--lr", "1e-2", "--cpu", "--distributed-world-size", "1",
                "--save-dir", str(tmp_path), "--disable-validation", "--log-format", "none", *extra]
        cfg = convert_namespace_to_config(options.parse_args_and_arch(options.get_training_parser(), input_args=argv))
        torch.manual_seed(1)
        task = tasks.setup_task(cfg.task)
        model, criterion = build_model_and_criterion(cfg, task)
        tr = Trainer(cfg, task, model, criterion)
        task.load_dataset("train")
        batch = task.dataset("train").collater([0, 1])
        norms = []
        for _ in range(3):
            tr.train_step([batch] * copies)
            norms.append(float(tr.last_grad_norm))
        return norms

    one, two = run(1), run(2)
    assert two == pytest.approx(one, rel=2e-2), (one, two)


def test_layers_grouped_into_one_sharded_unit_train_like_one_unit_per_layer(tmp_path):
    base = _run(tmp_path / "a", POLY + ["--ddp-backend", "fully_sharded"])
    grouped = _run(tmp_path / "b", POLY + ["--ddp-backend", "fully_sharded", "--fsdp-checkpoint-wrap-layer-frequency", "2"])
    assert grouped == pytest.approx(base, rel=1e-5)


def test_recomputing_the_modular_layer_gives_the_losses_of_keeping_its_activations(tmp_path):
    """With dropout on: the recomputation must replay the same masks, or the two trajectories drift apart."""
    flags = POLY + ["--no-fused-layer", "--dropout", "0.1"]
    kept = _run(tmp_path / "a", flags)
    recomputed = _run(tmp_path / "b", flags + ["--checkpoint-activations"])
    assert recomputed == pytest.approx(kept, rel=1e-5)
