"""EMA shadow model: follows the exponential recurrence over real training steps, is stored in and restored from
the checkpoint state, and can be swapped into the live model."""
import copy

import pytest
import torch

from metaseq_b200 import options, tasks
from metaseq_b200.cli.train import build_model_and_criterion
from metaseq_b200.dataclass.utils import convert_namespace_to_config
from metaseq_b200.trainer import Trainer


def _trainer(tmp_path, extra=()):
    argv = [
        "--task", "dummy_lm", "--dict-size", "60", "--tokens-per-sample", "16", "--batch-size", "2",
        "--arch", "transformer_lm_megatron", "--decoder-layers", "1", "--decoder-embed-dim", "32",
        "--decoder-ffn-embed-dim", "64", "--decoder-attention-heads", "2", "--dropout", "0.0", "--attention-dropout", "0.0",
        "--criterion", "cross_entropy", "--optimizer", "adam", "--lr", "1e-2", "--lr-scheduler", "polynomial_decay",
        "--warmup-updates", "1", "--total-num-update", "50", "--cpu", "--distributed-world-size", "1",
        "--save-dir", str(tmp_path), "--disable-validation", "--log-format", "none", *extra,
    ]
    cfg = convert_namespace_to_config(options.parse_args_and_arch(options.get_training_parser(), input_args=argv))
    torch.manual_seed(2)
    task = tasks.setup_task(cfg.task)
    model, criterion = build_model_and_criterion(cfg, task)
    tr = Trainer(cfg, task, model, criterion)
    task.load_dataset("train")
    return tr, task.dataset("train").collater([0, 1])


def test_ema_follows_the_recurrence_and_round_trips_through_the_checkpoint_state(tmp_path):
    decay = 0.8
    tr, batch = _trainer(tmp_path, ["--store-ema", "--ema-decay", str(decay), "--ema-fp32"])
    shadow = {k: v.detach().clone().float() for k, v in tr.get_model().state_dict().items() if v.is_floating_point()}
    for _ in range(4):
        tr.train_step([batch])
        live = tr.get_model().state_dict()
        for k in shadow:
            shadow[k] = decay * shadow[k] + (1 - decay) * live[k].detach().float()
    ema_state = tr.ema.get_model().state_dict()
    moved = 0
    for k, want in shadow.items():
        assert torch.allclose(ema_state[k].float(), want, atol=1e-5, rtol=1e-4), k
        moved += int(not torch.allclose(ema_state[k].float(), live[k].float(), atol=1e-6))
    assert moved > 0  # the shadow lags the live weights
    state = tr.state_dict()
    assert "ema" in state["extra_state"] and "ema_fp32_params" in state["extra_state"]
    # restore into a fresh shadow and swap it into a model
    tr2, _ = _trainer(tmp_path, ["--store-ema", "--ema-decay", str(decay), "--ema-fp32"])
    tr2.ema.restore(copy.deepcopy(state["extra_state"]["ema"]), build_fp32_params=True)
    for k, want in shadow.items():
        assert torch.allclose(tr2.ema.get_model().state_dict()[k].float(), want, atol=1e-5, rtol=1e-4)
    target = tr2.get_model()
    tr2.ema.reverse(target)
    for k, want in shadow.items():
        assert torch.allclose(target.state_dict()[k].float(), want, atol=1e-5, rtol=1e-4)


def test_ema_over_a_fully_sharded_model_averages_the_flat_shards(tmp_path):
    decay = 0.5
    tr, batch = _trainer(tmp_path, ["--store-ema", "--ema-decay", str(decay), "--ema-fp32", "--ddp-backend",
                                    "fully_sharded", "--use-sharded-state"])
    keys = [k for k in tr.get_model().state_dict() if k.endswith("flat_param_0")]
    assert keys, list(tr.get_model().state_dict())
    shadow = {k: tr.get_model().state_dict()[k].detach().clone().float() for k in keys}
    for _ in range(3):
        tr.train_step([batch])
        live = tr.get_model().state_dict()
        for k in keys:
            shadow[k] = decay * shadow[k] + (1 - decay) * live[k].detach().float()
    assert tr.ema.get_model() is not tr.get_model()
    ema_state = tr.ema.get_model().state_dict()
    for k in keys:
        assert torch.allclose(ema_state[k].float(), shadow[k], atol=1e-5, rtol=1e-4), k
        assert not torch.allclose(ema_state[k].float(), live[k].float(), atol=1e-7)


def test_ema_seed_model_and_update_frequency(tmp_path):
    tr, batch = _trainer(tmp_path, [])
    seed_state = {k: torch.full_like(v, 0.25) if v.is_floating_point() else v.clone()
                  for k, v in tr.get_model().state_dict().items()}
    seed_path = tmp_path / "seed.pt"
    torch.save({"model": {}, "extra_state": {"ema": seed_state}}, seed_path)
    tr2, batch = _trainer(tmp_path, ["--store-ema", "--ema-decay", "0.5", "--ema-seed-model", str(seed_path),
                                     "--ema-update-freq", "2"])
    start = tr2.ema.get_model().state_dict()
    name = next(k for k, v in start.items() if v.is_floating_point() and "version" not in k)
    assert torch.all(start[name] == 0.25)
    tr2.train_step([batch])  # first of two: no EMA update yet
    assert torch.all(tr2.ema.get_model().state_dict()[name] == 0.25)
    tr2.train_step([batch])
    want = 0.5 * 0.25 + 0.5 * tr2.get_model().state_dict()[name].float()
    assert torch.allclose(tr2.ema.get_model().state_dict()[name].float(), want, atol=1e-6)


def test_activation_norms_and_parameter_statistics_are_logged(tmp_path):
    from metaseq_b200.logging import metrics

    metrics.reset()
    tr, batch = _trainer(tmp_path, ["--criterion", "vocab_parallel_cross_entropy", "--ddp-backend", "fully_sharded",
                                    "--use-sharded-state", "--log-param-stats", "--decoder-learned-pos",
                                    "--no-scale-embedding"])
    out = tr.train_step([batch])
    model = tr.get_model()
    with torch.no_grad():
        tokens = batch["net_input"]["src_tokens"]
        dec = model.decoder
        tok = dec.embed_tokens.weight[tokens].float()
        want_tok = tok.norm(dim=-1).mean()
    for key in ("actv_norm", "emb_norm", "tok_norm", "pos_norm"):
        assert key in out and float(out[key]) > 0, (key, sorted(out))
    train = metrics.get_smoothed_values("train")
    stats = [k for k in train if k.startswith(("gnorm_", "gmax_", "gzero_", "pnorm_", "pmax_", "pzero_"))]
    assert {k.split("_")[0] for k in stats} == {"gnorm", "gmax", "gzero", "pnorm", "pmax", "pzero"}, sorted(train)
    # the token-embedding norm was taken before the update: compare with a tolerance that covers one Adam step
    assert float(out["tok_norm"]) == pytest.approx(float(want_tok), rel=0.2)
