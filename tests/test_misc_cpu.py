"""Small host-side components: utils, metrics / meters, module proxy, service queue and responses, sequence
generator on a scripted model, launcher, options -> config, NaN detector, file chunker."""
import json
import logging
import os

import pytest
import torch

from metaseq_b200 import utils
from metaseq_b200.logging import meters, metrics


# ------------------------------------------------------------------------------ utils
def test_make_positions_skips_padding_and_offsets_by_pad_index():
    pad = 1
    toks = torch.tensor([[9, 9, 9, 1, 1], [1, 1, 9, 9, 9], [9, 1, 9, 1, 9]])
    pos = utils.make_positions(toks, pad)
    assert pos.tolist() == [[2, 3, 4, 1, 1], [1, 1, 2, 3, 4], [2, 1, 3, 1, 4]]


def test_clip_grad_norm_scales_in_place_and_reports_total():
    params = [torch.nn.Parameter(torch.zeros(5)) for _ in range(3)]
    assert float(utils.clip_grad_norm_(params, 1.0)) == 0.0  # no gradients
    for p in params:
        p.grad = torch.full((5,), 2.0)
    total = utils.clip_grad_norm_(params, 1.0)
    assert float(total) == pytest.approx((15 * 4.0) ** 0.5)
    assert float(utils.clip_grad_norm_(params, 1.0)) == pytest.approx(1.0, rel=1e-5)
    for p in params:
        p.grad = torch.full((5,), 2.0)
    assert float(utils.clip_grad_norm_(params, 0.0)) == pytest.approx((15 * 4.0) ** 0.5)  # 0 = measure only
    assert params[0].grad[0].item() == 2.0
    params[1].grad[0] = 7.0
    assert float(utils.clip_grad_norm_(params, 0.0, norm_type="inf")) == 7.0


# --------------------------------------------------------------------- metrics / meters
def test_metrics_aggregators_nest_and_average():
    metrics.reset()
    with metrics.aggregate("train") as outer:
        metrics.log_scalar("loss", 2.0, weight=1)
        with metrics.aggregate("inner") as inner:
            metrics.log_scalar("loss", 4.0, weight=3)
        metrics.log_scalar_sum("n", 5)
        metrics.log_derived("double", lambda m: 2 * m["loss"].avg)
    assert inner.get_smoothed_value("loss") == 4.0
    assert outer.get_smoothed_value("loss") == pytest.approx((2.0 + 12.0) / 4)
    assert outer.get_smoothed_value("n") == 5
    assert outer.get_smoothed_value("double") == pytest.approx(7.0)
    state = metrics.state_dict()
    metrics.reset()
    metrics.load_state_dict(state)
    assert metrics.get_smoothed_value("train", "loss") == pytest.approx(3.5)


def test_meters_roundtrip_and_priority_order():
    d = meters.MetersDict()
    d.add_meter("late", meters.AverageMeter(round=2), priority=50)
    d.add_meter("early", meters.SumMeter(), priority=10)
    d.add_meter("derived", meters.MetersDict._DerivedMeter(lambda m: m["early"].sum + 1), priority=20)
    assert list(d.keys()) == ["early", "derived", "late"]
    d["late"].update(1.23456, n=2)
    d["early"].update(3)
    assert d.get_smoothed_values() == {"early": 3, "derived": 4, "late": 1.23}
    d2 = meters.MetersDict()
    d2.load_state_dict(d.state_dict())
    assert d2["late"].avg == pytest.approx(1.23456) and "derived" not in d2
    sw = meters.StopwatchMeter()
    sw.start()
    sw.stop(n=2)
    assert sw.n == 2 and sw.sum >= 0
    tm = meters.TimeMeter()
    tm.update(10)
    restored = meters.TimeMeter()
    restored.load_state_dict(tm.state_dict())
    assert restored.n == 10


def test_module_proxy_wrapper_forwards_attributes_and_state():
    from metaseq_b200.parallel.module_proxy_wrapper import ModuleProxyWrapper

    class Inner(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.linear = torch.nn.Linear(2, 2)
            self.custom = "x"

        def forward(self, x):
            return self.linear(x)

        def get_custom(self):
            return self.custom

    class FakeDDP(torch.nn.Module):
        def __init__(self, module):
            super().__init__()
            self.module = module
            self.ddp_only = 3

        def forward(self, x):
            return self.module(x)

    inner = Inner()
    wrapped = ModuleProxyWrapper(FakeDDP(inner))
    assert wrapped.get_custom() == "x" and wrapped.ddp_only == 3 and wrapped.linear is inner.linear
    assert set(wrapped.state_dict().keys()) == {"linear.weight", "linear.bias"}
    with pytest.raises(AttributeError):
        wrapped.nope
    with pytest.raises(AssertionError):
        ModuleProxyWrapper(inner)
    x = torch.randn(3, 2)
    assert torch.equal(wrapped(x), inner(x))


# ------------------------------------------------------------------------------ service
def test_service_queue_batches_compatible_requests_cheapest_first():
    from metaseq_b200.service.queue import PriorityQueueRing
    from metaseq_b200.service.workers import WorkItem

    ring = PriorityQueueRing(num_shards=2)
    for uid, (cost, temp) in enumerate([(30, 1.0), (10, 1.0), (20, 0.7), (5, 1.0)]):
        ring.put(WorkItem(cost=cost, uid=uid, return_queue=None, data={"input": [1], "temperature": temp, "n": 1}))
    assert not ring.empty()
    seen = []
    while not ring.empty():
        shard = ring.largest_shard()
        q = shard.get_deepest_queue() if hasattr(shard, "get_deepest_queue") else shard
        item = shard.get()
        seen.append((item.cost, item.data["temperature"]))
    assert sorted(seen) == [(5, 1.0), (10, 1.0), (20, 0.7), (30, 1.0)]
    same_key = [c for c, t in seen if t == 1.0]
    assert same_key == sorted(same_key)  # within one sampling configuration the cheapest request comes first


def test_oai_response_envelope():
    from metaseq_b200.service.responses import OAIResponse

    r = OAIResponse([{"text": "hi", "tokens": ["h", "i"], "token_scores": [-0.1, -0.2], "text_offset": [0, 1],
                      "top_logprobs": None}]).__dict__()
    assert r["object"] == "text_completion" and r["choices"][0]["text"] == "hi"
    assert r["choices"][0]["logprobs"]["token_logprobs"] == [-0.1, -0.2]
    json.dumps(r)


def test_service_newline_normalisation():
    from metaseq_b200.service.utils import normalize_newlines

    assert normalize_newlines("a\r\nb\rc\n") == "a\nb\nc\n"


# ------------------------------------------------------------------- sequence generator
class ScriptedDecoder(torch.nn.Module):
    """Next-token distribution depends only on the last token: t -> t + 1 (mod V), EOS after token 7."""

    def __init__(self, vocab, eos):
        super().__init__()
        self.vocab, self.eos = vocab, eos
        self.calls = []

    def forward(self, tokens, incremental_state=None, **kw):
        self.calls.append(tokens.shape[1])
        nxt = torch.where(tokens == 7, torch.full_like(tokens, self.eos), (tokens + 1) % self.vocab)
        logits = torch.full((*tokens.shape, self.vocab), -10.0)
        logits.scatter_(-1, nxt.unsqueeze(-1), 10.0)
        return logits, None


class ScriptedModel(torch.nn.Module):
    def __init__(self, vocab, eos):
        super().__init__()
        self.decoder = ScriptedDecoder(vocab, eos)

    def forward(self, tokens, **kw):
        return self.decoder(tokens, **kw)

    def max_decoder_positions(self):
        return 32


def test_sequence_generator_greedy_follows_the_model_and_stops_at_eos():
    from metaseq_b200.data import Dictionary
    from metaseq_b200.sequence_generator import SequenceGenerator

    d = Dictionary()
    for i in range(12):
        d.add_symbol(str(i))
    gen = SequenceGenerator(ScriptedModel(len(d), d.eos()), d, beam_size=1, max_len_b=20, temperature=1.0, topp=-1.0,
                            sampling=False) if "sampling" in SequenceGenerator.__init__.__code__.co_varnames else \
        SequenceGenerator(ScriptedModel(len(d), d.eos()), d, beam_size=1, max_len_b=20, topp=-1.0)
    src = torch.tensor([[d.eos(), 4, 5], [d.eos(), 6, d.pad()]])
    out = gen._generate({"net_input": {"src_tokens": src}})
    toks = out["tokens"][:, 0]
    assert toks[0, :6].tolist() == [d.eos(), 4, 5, 6, 7, d.eos()]
    # the second prompt is one token shorter: generation continues from its own last real token
    assert toks[1, :2].tolist() == [d.eos(), 6] and 7 in toks[1].tolist()
    assert out["scores"].shape == out["tokens"].shape


# ------------------------------------------------------------------------------ launcher
def test_launcher_grid_expands_to_one_command_per_combination(tmp_path, capsys):
    from metaseq_b200.launcher import slurm, sweep

    def get_grid(args):
        return [sweep.hyperparam("--lr", [0.1, 0.2], save_dir_key=lambda v: f"lr{v}"),
                sweep.hyperparam("--fp16", binary_flag=True, values=True),
                sweep.hyperparam("--seed", 3)]

    args = sweep.get_args(input_args=["-p", "exp", "-g", "2", "-n", "1", "--dry-run", "--local", "--checkpoints-dir",
                                      str(tmp_path)])
    dirs = slurm.main(get_grid, lambda a, c: None, args)
    out = capsys.readouterr().out
    assert len(dirs) == 2 and any(d.endswith("exp.lr0.1.ngpu2") for d in dirs)
    assert out.count("train command:") == 2 and "--lr 0.2 --fp16 --seed 3" in out
    with pytest.raises(ValueError):
        sweep.hyperparam("--x", [1, 2])  # several values need a save_dir_key


def test_launcher_skips_finished_runs_and_builds_sbatch(tmp_path):
    from metaseq_b200.launcher import slurm, sweep

    args = sweep.get_args(input_args=["-p", "exp", "-g", "8", "-n", "2", "--checkpoints-dir", str(tmp_path),
                                      "--partition", "learn", "--time", "60"])
    done = tmp_path / "run"
    done.mkdir()
    (done / "train.log").write_text("step 1\ndone training in 3 seconds\n")
    assert slurm.is_finished(str(done)) and not slurm.is_job_valid(args, str(done), lambda m: False)
    cmd, text = slurm.gen_sbatch_command_and_str(args, "job", "log", "err", "", "srun python x")
    assert "--signal" in cmd and "B:USR1@180" in cmd and "--partition" in cmd
    assert "scontrol requeue $SLURM_JOB_ID" in cmd[-1]
    env = {}
    slurm.set_env(args, env, lambda m: False)
    assert env["NCCL_ASYNC_ERROR_HANDLING"] == "1"


def test_launcher_cluster_flags_data_and_upload_paths(tmp_path, capsys):
    from metaseq_b200.launcher import slurm, sweep

    def get_grid(args):
        return [sweep.hyperparam("--lr", [0.1], save_dir_key=lambda v: f"lr{v}")]

    base = ["-p", "exp", "-g", "2", "-n", "1", "--dry-run", "--local", "--checkpoints-dir", str(tmp_path)]
    args = sweep.get_args(input_args=base + ["--azure", "-d", "/data/corpus", "--local-checkpoints-dir", "/mnt/scratch",
                                             "--full-azure-upload-path", "https://acct.blob.example/cont/run?sig=abc",
                                             "--azure-folder-auto-name"])
    assert args.cluster_env == "azure"
    slurm.main(get_grid, lambda a, c: None, args)
    out = capsys.readouterr().out
    line = next(ln for ln in out.splitlines() if "train command:" in ln)
    assert " /data/corpus " in line
    assert "--save-dir /mnt/scratch/exp.lr0.1.ngpu2" in line
    assert "--save-async --cloud-upload-path 'https://acct.blob.example/cont/run/exp.lr0.1.ngpu2/?sig=abc'" in line
    # without the auto-name flag the URL is passed through; without a local dir the save dir is the job's own
    args = sweep.get_args(input_args=base + ["--fair", "--full-azure-upload-path", "nfs:/shared/ckpt"])
    assert args.cluster_env == "fair"
    slurm.main(get_grid, lambda a, c: None, args)
    line = next(ln for ln in capsys.readouterr().out.splitlines() if "train command:" in ln)
    assert f"--save-dir {tmp_path}/exp.lr0.1.ngpu2" in line and "--cloud-upload-path nfs:/shared/ckpt" in line
    with pytest.raises(SystemExit):
        sweep.get_args(input_args=base + ["--aws", "--rsc"])


def test_tombstone_triggers_action_and_is_removed(tmp_path):
    from metaseq_b200.launcher.tombyard import tombstones, tombstones_procedure

    fired = []
    actions = {k: (lambda k=k: fired.append(k)) for k in ("scancel", "requeuehold", "release")}
    assert tombstones_procedure("42", str(tmp_path), period=0.0, actions=actions, max_polls=2) is None and not fired
    open(tombstones("42", str(tmp_path))["scancel"], "w").close()
    assert tombstones_procedure("42", str(tmp_path), period=0.0, actions=actions, max_polls=2) == "scancel"
    assert fired == ["scancel"] and not os.path.exists(tombstones("42", str(tmp_path))["scancel"])


def test_opt_baselines_grid_matches_model_table():
    from metaseq_b200.launcher import opt_baselines, sweep
    from metaseq_b200.launcher.opt_job_constants import MODEL_SIZES

    args = sweep.get_args(opt_baselines.add_extra_options_func,
                          ["-p", "t", "-g", "8", "--model-size", "1.3b", "--benchmark", "--local", "--dry-run"])
    grid = {h.name: h for h in opt_baselines.get_grid(args)}
    size = MODEL_SIZES["1.3b"]
    assert grid["--decoder-layers"].values == [size.n_layers] and grid["--decoder-embed-dim"].values == [size.emb_size]
    assert grid["--task"].values == ["dummy_lm"] and grid["--max-update"].values == [50]
    assert grid["--model-parallel-size"].values == [size.model_parallel]
    assert grid["--lr"].values == [size.lr] and "--no-reshard-after-forward" in grid


# ------------------------------------------------------------------------ options / config
def test_training_parser_builds_nested_config_with_arch_defaults():
    from metaseq_b200 import options
    from metaseq_b200.dataclass.utils import convert_namespace_to_config

    parser = options.get_training_parser()
    ns = options.parse_args_and_arch(parser, input_args=[
        "--task", "dummy_lm", "--arch", "opt_125m", "--optimizer", "adam", "--lr", "3e-4", "--lr-scheduler",
        "polynomial_decay", "--total-num-update", "10", "--criterion", "cross_entropy", "--batch-size", "2",
        "--tokens-per-sample", "64", "--adam-betas", "(0.9, 0.95)", "--memory-efficient-fp16", "--model-parallel-size", "1"])
    cfg = convert_namespace_to_config(ns)
    assert cfg.common.memory_efficient_fp16 and cfg.common.fp16
    assert cfg.optimizer._name == "adam" and cfg.optimizer.adam_betas == "(0.9, 0.95)"
    assert cfg.lr_scheduler._name == "polynomial_decay" and cfg.task._name == "dummy_lm"
    assert cfg.model.decoder_layers == 12 and cfg.model.decoder_embed_dim == 768  # from the architecture function
    assert cfg.dataset.batch_size == 2 and cfg.optimization.lr == [3e-4]


# ---------------------------------------------------------------------------- nan detector
def test_nan_detector_names_the_first_bad_module(caplog):
    from metaseq_b200.nan_detector import NanDetector

    class Bad(torch.nn.Module):
        def forward(self, x):
            return x / 0.0 * 0.0

    model = torch.nn.Sequential(torch.nn.Linear(4, 4), Bad(), torch.nn.Linear(4, 4))
    with caplog.at_level(logging.WARNING, logger="metaseq_b200.nan_detector"):
        with NanDetector(model, backward=False) as det:
            model(torch.ones(2, 4))
    assert det.has_printed_f
    assert any("NaN detected in output of 1" in r.getMessage() for r in caplog.records)


def test_rms_norm_cpu_matches_definition():
    from metaseq_b200.modules.layer_norm import RMSNorm

    torch.manual_seed(0)
    mod = RMSNorm(48)
    with torch.no_grad():
        mod.weight.copy_(torch.randn(48))
    x = torch.randn(7, 48, requires_grad=True)
    y = mod(x)
    ref_in = x.detach().clone().requires_grad_(True)
    ref = ref_in * torch.rsqrt(ref_in.pow(2).mean(-1, keepdim=True) + mod.eps) * mod.weight.detach()
    dy = torch.randn(7, 48)
    y.backward(dy)
    ref.backward(dy)
    assert torch.allclose(y, ref, atol=1e-5) and torch.allclose(x.grad, ref_in.grad, atol=1e-5)
    want = (dy * ref_in.detach() * torch.rsqrt(ref_in.detach().pow(2).mean(-1, keepdim=True) + mod.eps)).sum(0)
    assert torch.allclose(mod.weight.grad, want, atol=1e-4)



def test_top_p_sampling_restatement_draws_from_the_nucleus():
    from metaseq_b200.ops import functional as F

    torch.manual_seed(0)
    lp = torch.log_softmax(torch.randn(4, 50) * 2, -1)
    lp[:, 3] = float("-inf")
    chosen_lp, tok = F.sample_top_p(lp, 1e-6)
    assert torch.equal(tok, lp.argmax(-1)) and torch.equal(chosen_lp, lp.max(-1).values)
    counts = torch.zeros(50)
    for _ in range(3000):
        _, t = F.sample_top_p(lp[:1], 0.8)
        counts[t[0]] += 1
    p = lp[0].exp()
    sp, si = p.sort(descending=True)
    keep = (sp.cumsum(0) - sp) < 0.8
    nucleus = si[keep]
    expect = torch.zeros(50)
    expect[nucleus] = p[nucleus] / p[nucleus].sum()
    assert counts[expect == 0].sum() == 0
    assert (counts / 3000 - expect).abs().max() < 0.03
    # one nucleus size per row
    _, t = F.sample_top_p(lp, torch.tensor([1e-6, 1e-6, 1e-6, 1e-6]))
    assert torch.equal(t, lp.argmax(-1))


def test_sampling_with_min_len_equal_to_max_len_ends_in_eos():
    """The last position forces EOS even when ``min_len`` still bans it, and a row whose tokens are all banned
    never reaches multinomial as an all-zero distribution."""
    from metaseq_b200.data import Dictionary
    from metaseq_b200.sequence_generator import SequenceGenerator

    d = Dictionary()
    for i in range(12):
        d.add_symbol(str(i))
    torch.manual_seed(0)
    gen = SequenceGenerator(ScriptedModel(len(d), d.eos()), d, beam_size=2, max_len_b=10, min_len=10, temperature=1.0,
                            topp=0.9)
    src = torch.tensor([[d.eos(), 4, 5]])
    out = gen._generate({"net_input": {"src_tokens": src}})
    toks = out["tokens"][0]
    assert toks.shape == (2, 10)
    assert (toks[:, -1] == d.eos()).all() and (toks[:, 3:-1] != d.eos()).all()
    all_banned = torch.full((3, len(d)), float("-inf"))
    lp, tok = gen._sample(all_banned)
    assert tok.shape == (3,)


def test_graphed_decode_step_declines_models_it_cannot_serve():
    """On a CPU (or any decoder that is not the framework's own) the generator keeps the module path."""
    from metaseq_b200.models.decode_step import GraphedDecodeStep
    from metaseq_b200.ops import functional as F

    assert not GraphedDecodeStep.supported(ScriptedDecoder(16, 2))
    with F.dependent_launch():  # no kernels library needed on a CPU: the context is a no-op
        pass

    from metaseq_b200 import options, tasks
    from metaseq_b200.dataclass.utils import convert_namespace_to_config

    parser = options.get_training_parser()
    ns = options.parse_args_and_arch(parser, input_args=[
        "--task", "dummy_lm", "--dict-size", "60", "--tokens-per-sample", "16", "--batch-size", "1",
        "--arch", "transformer_lm_megatron", "--decoder-layers", "1", "--decoder-embed-dim", "32",
        "--decoder-ffn-embed-dim", "64", "--decoder-attention-heads", "2", "--criterion", "cross_entropy",
        "--optimizer", "adam", "--lr", "1e-3", "--distributed-world-size", "1", "--cpu"])
    cfg = convert_namespace_to_config(ns)
    task = tasks.setup_task(cfg.task)
    model = task.build_model(cfg.model).eval()
    assert not GraphedDecodeStep.supported(model.decoder)


def test_service_launch_args_parse_and_data_may_be_positional():
    from metaseq_b200 import options
    from metaseq_b200.service import constants as C

    flat = []
    for s in C.LAUNCH_ARGS:
        flat += s.split()
    args = options.parse_args_and_arch(options.get_generation_parser(), input_args=flat)
    assert args.bpe == "hf_byte_bpe" and args.bpe_merges == C.BPE_MERGES and args.bpe_vocab == C.BPE_VOCAB
    assert args.data == "/tmp" and not hasattr(args, "data_positional")
    assert args.model_parallel_size == C.MODEL_PARALLEL

    parser = options.get_training_parser()
    base = ["--task", "streaming_language_modeling", "--arch", "transformer_lm_megatron", "--criterion", "cross_entropy",
            "--optimizer", "adam", "--lr", "1e-3", "--batch-size", "1", "--tokens-per-sample", "16"]
    a = options.parse_args_and_arch(parser, input_args=["/corpus"] + base)
    b = options.parse_args_and_arch(options.get_training_parser(), input_args=base + ["--data", "/corpus"])
    assert a.data == b.data == "/corpus"


def test_launcher_tells_failed_runs_from_running_ones(tmp_path):
    from metaseq_b200.launcher import slurm, sweep

    base = ["-p", "exp", "-g", "1", "--checkpoints-dir", str(tmp_path)]
    plain, resume = sweep.get_args(input_args=base), sweep.get_args(input_args=base + ["--resume-failed"])
    said = []
    run = tmp_path / "run"
    run.mkdir()
    assert slurm.is_job_valid(plain, str(run), said.append)  # nothing there yet
    (run / "train.log").write_text("step 1\n")
    assert slurm.has_started(str(run)) and not slurm.has_failed(str(run))
    assert not slurm.is_job_valid(plain, str(run), said.append)   # in progress
    assert not slurm.is_job_valid(resume, str(run), said.append)  # --resume-failed does not touch a healthy run
    (run / "train.stderr.7").write_text("Traceback ...\n")
    (run / "train.stderr.9").write_text("\n  \n")
    assert not slurm.has_failed(str(run))                         # the newest job's stderr is blank
    (run / "train.stderr.12").write_text("RuntimeError: boom\n")
    assert slurm.has_failed(str(run))
    assert not slurm.is_job_valid(plain, str(run), said.append)
    assert slurm.is_job_valid(resume, str(run), said.append) and any("resume failed run" in m for m in said)
    (run / "train.log").write_text("step 1\ndone training in 3 s\n")
    assert slurm.has_finished(str(run)) and not slurm.is_job_valid(resume, str(run), said.append)
    log = tmp_path / "git.log"
    log.write_text("")
    slurm.write_git_commit(str(log))
    assert log.read_text() == "" or log.read_text().startswith("commit ")


def test_fsdp_reshard_functions_work_on_state_dicts_in_memory():
    """Two shards of one flat parameter (two tensors, padded) -> three shards -> one unflattened dict."""
    from metaseq_b200.checkpoint import flat_shards, reshard_fsdp

    a, b = torch.arange(6.0).view(2, 3), torch.arange(6.0, 11.0)
    full = torch.cat([a.flatten(), b])
    per = flat_shards.shard_size_for(full.numel(), 2)
    padded = torch.cat([full, torch.zeros(2 * per - full.numel())])

    def shard(r):
        pad = max(0, min(per, (r + 1) * per - full.numel()))
        md = {"param_metadata": [{"fsdp_path": "decoder", "params": {"flat_param_0": {
            "names": ["w", "v"], "shapes": [[2, 3], [5]], "numels": [6, 5], "padding": pad}},
            "no_broadcast_optim_state": False, "shared_param_info": []}], "buffer_names": []}
        piece = padded[r * per:(r + 1) * per].clone()
        return {"model": {"decoder.flat_param_0": piece, "decoder.version": torch.tensor([3.0])}, "shard_metadata": md,
                "last_optimizer_state": {"state": {0: {"step": 4, "exp_avg": piece * 0.5}}, "param_groups": [{"lr": 0.1}]},
                "cfg": {"x": 1}, "extra_state": {"train_iterator": {"tokenization_cache": b"big", "epoch": 2}}}

    three = reshard_fsdp.reshard_fsdp_state_dicts([shard(0), shard(1)], num_output_shards=3, unflatten_weights=False,
                                                  dtype=torch.float16, drop_metaseq_req=True)
    assert len(three) == 3 and all(s["cfg"] == {"x": 1} and s["extra_state"]["train_iterator"] is None for s in three)
    assert all(s["model"]["decoder.flat_param_0"].dtype == torch.float16 for s in three)
    assert three[0]["last_optimizer_state"]["state"][0]["step"] == 4
    back = reshard_fsdp.reshard_fsdp_state_dicts(three, num_output_shards=1, unflatten_weights=True)
    assert set(back[0]) == {"model", "cfg", "extra_state"}
    assert torch.equal(back[0]["model"]["decoder.w"].float(), a) and torch.equal(back[0]["model"]["decoder.v"].float(), b)
    opt = reshard_fsdp.reshard_fsdp_optim_state(
        [s["last_optimizer_state"] for s in three], [s["shard_metadata"] for s in three],
        [s["model"] for s in three], num_output_shards=1)
    assert torch.allclose(opt[0]["state"][0]["exp_avg"][:11].float(), full * 0.5)
    with pytest.raises(ValueError, match="Unflatten weights only"):
        reshard_fsdp.reshard_fsdp_model_weights([shard(0)["model"]], [shard(0)["shard_metadata"]], 2, True)


def test_stitching_functions_consolidate_parts_and_recut_the_fused_projection(tmp_path):
    from metaseq_b200.checkpoint import consolidate_fsdp_shards as cons
    from metaseq_b200.checkpoint import reshard_consolidated, reshard_mp

    torch.manual_seed(0)
    D = 4
    full = {"decoder.layers.0.self_attn.qkv_proj.weight": torch.randn(3 * D, D),
            "decoder.layers.0.fc2.weight": torch.randn(D, 2 * D), "decoder.layers.0.fc2.bias": torch.randn(D),
            "decoder.embed_tokens.weight": torch.randn(8, D)}
    parts = reshard_mp.reshard_megatron_parts([full], new_model_part_count=2)
    ks, vs, qs = cons.handle_qkv_proj(parts, "decoder.layers.0.self_attn.qkv_proj.weight", 1)
    assert torch.equal(torch.cat([ks[0], vs[0], qs[0]]), full["decoder.layers.0.self_attn.qkv_proj.weight"])

    # every part as two flat shards, then back through consolidate_model_parallel
    weights, metadata, names = [], [], []
    for p, part in enumerate(parts):
        md = {"param_metadata": [{"fsdp_path": "", "params": {"flat_param_0": {
            "names": list(part), "shapes": [list(t.shape) for t in part.values()],
            "numels": [t.numel() for t in part.values()], "padding": 0}},
            "no_broadcast_optim_state": False, "shared_param_info": []}], "buffer_names": []}
        w, m = reshard_consolidated.reshard_unflattened_model_weights(dict(part), md, 2)
        for r in range(2):
            weights.append(w[r])
            metadata.append(m[r])
            names.append(f"ckpt-model_part-{p}-shard{r}.pt")
    glued = cons.consolidate_model_parallel(metadata, names, True, weights, parts=2)
    assert set(glued) == set(full) and all(torch.equal(glued[k], full[k]) for k in full)
    kept = cons.consolidate_model_parallel(metadata, names, True, weights, parts=2, no_stitch_megatron=True)
    assert sorted(kept) == [0, 1] and torch.equal(kept[1]["decoder.layers.0.fc2.weight"], parts[1]["decoder.layers.0.fc2.weight"])

    # the file-level entry points under the reference's names
    for p, part in enumerate(parts):
        torch.save({"model": part, "cfg": {"model": {"model_parallel_size": 2}}}, tmp_path / f"in-model_part-{p}.pt")
    out = reshard_mp.reshard_model_parallel_parts(str(tmp_path / "in-model_part-*.pt"), str(tmp_path / "one-{i}.pt"), 1)
    one = torch.load(out[0], weights_only=False)
    assert all(torch.equal(one["model"][k], full[k]) for k in full) and one["cfg"]["model"]["model_parallel_size"] == 1
    with pytest.raises(ValueError, match="doesn't match any"):
        reshard_mp.reshard_model_parallel_parts(str(tmp_path / "none-*.pt"), str(tmp_path / "x-{i}.pt"))


def test_int8_weight_only_quantize_fills_the_four_matrix_slots():
    from metaseq_b200.checkpoint import convert_metaseq_ft as ft

    n = 2
    weights = [torch.randn(6, 3, 4) if slot == 2 else torch.randn(6, 8) for slot in range(12) for _ in range(n)]
    kept = [w.clone() for w in weights]
    q, s = ft.int8_weight_only_quantize(weights, n)
    assert len(q) == len(s) == 4 * n and all(t.dtype == torch.int8 for t in q)
    w0 = kept[2 * n].flatten(1)
    assert torch.allclose(q[0].float() * s[0], w0, atol=float(w0.abs().max()) / 127 + 1e-6)
    assert weights[2 * n].numel() == 0 and weights[0].numel() > 0


def test_generation_config_is_inferred_from_a_checkpoint_directory(tmp_path):
    from metaseq_b200.checkpoint.convert_to_singleton import create_generation_config_with_defaults

    for p in range(2):
        (tmp_path / f"reshard-model_part-{p}.pt").write_bytes(b"")
    cfg = create_generation_config_with_defaults(str(tmp_path))
    assert cfg.common.model_parallel_size == 2 and cfg.distributed_training.distributed_world_size == 2
    assert cfg.common_eval.path == str(tmp_path / "reshard.pt")
    assert cfg.task.vocab_filename == str(tmp_path / "gpt2-vocab.json")
    (tmp_path / "gpt2-unified.json").write_text("{}")
    cfg = create_generation_config_with_defaults(str(tmp_path))
    assert cfg.task.hf_tokenizer == str(tmp_path / "gpt2-unified.json")


def test_launcher_helpers_name_the_run_snapshot_sources_and_pick_the_cluster(tmp_path):
    import types

    from metaseq_b200.launcher import slurm, sweep
    from metaseq_b200.launcher.opt_job_constants import ComputeEnvs

    said = []
    args = types.SimpleNamespace(checkpoints_dir=str(tmp_path), prefix="exp", num_nodes=2, num_gpus=8)
    config = {"--lr": sweep.hyperparam("--lr", [0.1], save_dir_key=lambda v: f"lr{v}"),
              "--fp16": sweep.hyperparam("--fp16", binary_flag=True)}
    for hp in config.values():
        hp.current_value = hp.values[0]
    key, save_dir = slurm.run_setup(args, config, lambda msg: said.append(msg) or True)
    assert key == "lr0.1" and save_dir == str(tmp_path / "exp.lr0.1.ngpu16") and not os.path.exists(save_dir)
    key, save_dir = slurm.run_setup(args, config, lambda msg: False)
    assert os.path.isdir(save_dir)

    src = tmp_path / "src"
    (src / "pkg" / "sub").mkdir(parents=True)
    (src / "setup.py").write_text("x")
    (src / "notes.txt").write_text("x")
    (src / "pkg" / "a.py").write_text("x")
    (src / "pkg" / "sub" / "k.cu").write_text("x")
    (src / "pkg" / "sub" / "big.bin").write_text("x")
    dst = slurm.copy_all_python_files(str(src), str(tmp_path / "snap"), "abc123", recurse_dirs="pkg")
    got = sorted(os.path.relpath(os.path.join(d, f), dst) for d, _, fs in os.walk(dst) for f in fs)
    assert got == ["pkg/a.py", "pkg/sub/k.cu", "setup.py"]

    assert "export NCCL_TOPO_FILE=/opt/microsoft/ndv4-topo.xml" in slurm.azure_support()
    out = slurm.dry_run_batch({}, "log", "err", "no-such-sbatch x", ["no-such-sbatch", "x"], lambda m: said.append(m) or True)
    assert out is None and "- run command: no-such-sbatch x" in said

    ns = types.SimpleNamespace(azure=False, aws=True, fair=False, rsc=False)
    assert sweep.get_env_from_args(ns) == ComputeEnvs.AWS
    with pytest.raises(NotImplementedError):
        sweep.get_env_from_args(types.SimpleNamespace(azure=False, aws=False, fair=False, rsc=False))


def test_checkpoint_tools_take_the_reference_argument_spellings(tmp_path):
    """``--input / --output``, underscores for dashes, and booleans with an explicit value, as python-fire takes them."""
    import argparse

    from metaseq_b200.checkpoint import reshard_mp
    from metaseq_b200.checkpoint._cli import add_option, add_switch

    ap = argparse.ArgumentParser()
    add_option(ap, "--src-dir-pattern", "--input", dest="src")
    add_option(ap, "--num-output-shards", type=int, default=1)
    add_switch(ap, "--unflatten-weights")
    add_switch(ap, "--skip-optimizer-state")
    a = ap.parse_args(["--input", "x*.pt", "--num_output_shards", "2", "--unflatten-weights", "True",
                       "--skip_optimizer_state=False"])
    assert (a.src, a.num_output_shards, a.unflatten_weights, a.skip_optimizer_state) == ("x*.pt", 2, True, False)
    assert ap.parse_args(["--src-dir-pattern", "y", "--unflatten-weights"]).unflatten_weights is True
    with pytest.raises(SystemExit):
        ap.parse_args(["--unflatten-weights", "maybe"])

    torch.save({"model": {"decoder.layers.0.fc1.weight": torch.ones(4, 2)}, "cfg": {}}, tmp_path / "in-model_part-0.pt")
    reshard_mp.main(["--input", str(tmp_path / "in-model_part-*.pt"), "--output", str(tmp_path / "out-{i}.pt"),
                     "--num_output_parts", "2"])
    assert torch.load(tmp_path / "out-1.pt", weights_only=False)["model"]["decoder.layers.0.fc1.weight"].shape == (2, 2)
