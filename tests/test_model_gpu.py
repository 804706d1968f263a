"""GPU tests of the model-level paths: the fused decoder layer against the modular PyTorch
layer, a short fp16 training run with the kernels against the same run on the cuBLAS / PyTorch
backend, FSDP gradient plumbing, and incremental decoding against full re-computation."""
import copy
import math

import pytest
import torch

from metaseq_b200 import options, tasks
from metaseq_b200.cli.train import build_model_and_criterion
from metaseq_b200.dataclass.utils import convert_namespace_to_config
from metaseq_b200.ops import _lib
from metaseq_b200.ops import functional as F
from metaseq_b200.trainer import Trainer

pytestmark = pytest.mark.gpu


def _cfg(extra=(), fsdp=True, layers=2, dim=256, heads=4, seq=256, bsz=2):
    argv = [
        "--task", "dummy_lm", "--dict-size", "50272", "--tokens-per-sample", str(seq), "--batch-size", str(bsz),
        "--arch", "opt_125m", "--decoder-layers", str(layers), "--decoder-embed-dim", str(dim),
        "--decoder-attention-heads", str(heads), "--decoder-ffn-embed-dim", str(4 * dim), "--dropout", "0.0",
        "--attention-dropout", "0.0", "--criterion", "vocab_parallel_cross_entropy", "--optimizer", "adam",
        "--adam-betas", "(0.9, 0.95)", "--weight-decay", "0.1", "--clip-norm", "1.0", "--lr", "1e-3",
        "--lr-scheduler", "polynomial_decay", "--warmup-updates", "2", "--total-num-update", "100",
        "--memory-efficient-fp16", "--fp16-init-scale", "4", "--distributed-world-size", "1",
        "--save-dir", "/tmp/msq_test_gpu", "--disable-validation", "--log-format", "none",
        "--tensor-parallel-init-model-on-gpu",
    ]
    if fsdp:
        argv += ["--ddp-backend", "fully_sharded", "--use-sharded-state", "--no-reshard-after-forward",
                 "--min-params-to-wrap", "1000"]
    argv += list(extra)
    parser = options.get_training_parser()
    return convert_namespace_to_config(options.parse_args_and_arch(parser, input_args=argv))


def _trainer(cfg, seed=3):
    torch.manual_seed(seed)
    torch.cuda.manual_seed(seed)
    task = tasks.setup_task(cfg.task)
    model, criterion = build_model_and_criterion(cfg, task)
    tr = Trainer(cfg, task, model, criterion)
    task.load_dataset("train")
    return tr, task.dataset("train").collater([0])


def test_fused_layer_matches_modular_layer():
    cfg = _cfg(fsdp=False, layers=1)
    tr, batch = _trainer(cfg)
    layer = tr.get_model().decoder.layers[0]
    B, T, D = 2, 256, 256
    x = (torch.randn(B, T, D, device="cuda") * 0.5).half().requires_grad_(True)
    dy = torch.randn(B, T, D, device="cuda").half()
    assert layer._fused_ok(x, None, None, None)
    y = layer(x)
    y.backward(dy)
    g_fused = {n: p.grad.clone() for n, p in layer.named_parameters()}
    dx_fused = x.grad.clone()
    x.grad = None
    for p in layer.parameters():
        p.grad = None
    F.set_backend("torch")
    try:
        layer.use_fused_layer = False
        y2 = layer(x)
        y2.backward(dy)
    finally:
        F.set_backend("auto")
        layer.use_fused_layer = True
    torch.testing.assert_close(y.float(), y2.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dx_fused.float(), x.grad.float(), rtol=3e-2, atol=3e-2)
    for n, p in layer.named_parameters():
        ref = p.grad.float()
        got = g_fused[n].float()
        scale = max(1.0, float(ref.abs().max()))
        assert float((got - ref).abs().max()) / scale < 5e-2, n
    assert _lib.check_status("cuda") == 0


def test_training_kernels_match_torch_backend():
    losses = {}
    for backend in ("auto", "torch"):
        F.set_backend(backend)
        try:
            tr, batch = _trainer(_cfg(extra=["--kernel-backend", backend]))
            F.set_backend(backend)
            out = []
            for _ in range(6):
                log = tr.train_step([batch])
                if log is not None:
                    out.append(float(log["loss"]))
            losses[backend] = out
        finally:
            F.set_backend("auto")
    assert len(losses["auto"]) >= 4
    n = min(len(losses["auto"]), len(losses["torch"]))
    for a, b in zip(losses["auto"][:n], losses["torch"][:n]):
        assert abs(a - b) < 0.05, (losses["auto"], losses["torch"])
    # random labels on a fixed batch: the loss must go down as the model memorises it
    assert losses["auto"][-1] < losses["auto"][0]
    assert _lib.check_status("cuda") == 0


def test_fsdp_flat_grads_equal_plain_grads():
    tr_f, batch = _trainer(_cfg(fsdp=True))
    tr_p, _ = _trainer(_cfg(fsdp=False))
    sample = tr_f._prepare_sample(batch)[0]
    for tr in (tr_f, tr_p):
        tr.model.train()
        tr.zero_grad()
        loss, _, _ = tr.criterion(tr.model, sample)
        loss.backward()
    plain = dict(tr_p.get_model().named_parameters())
    model = tr_f.model
    for path, unit in model._unit_paths():
        flat_g = unit.flat_param.grad
        assert flat_g is not None, path
        off = 0
        for name, shape, n in zip(unit.param_names, unit.param_shapes, unit.param_numels):
            key = f"{path}.{name}" if path else name
            ref = plain[key].grad.float()
            got = flat_g[off:off + n].view(shape).float()
            scale = max(1.0, float(ref.abs().max()))
            assert float((got - ref).abs().max()) / scale < 5e-2, key
            off += n


def test_incremental_decoding_matches_full_forward():
    cfg = _cfg(fsdp=False)
    tr, batch = _trainer(cfg)
    model = tr.get_model().eval()
    tokens = torch.randint(4, 50272, (2, 40), device="cuda")
    with torch.no_grad():
        full, _ = model(tokens)
        state = {}
        step_logits = []
        out, _ = model(tokens[:, :32], incremental_state=state)
        step_logits.append(out[:, -1])
        for t in range(32, 39):
            out, _ = model(tokens[:, : t + 1], incremental_state=state)
            assert out.shape[1] == 1
            step_logits.append(out[:, -1])
    for i, t in enumerate(range(31, 39)):
        torch.testing.assert_close(step_logits[i].float(), full[:, t].float(), rtol=5e-2, atol=5e-2)
        assert torch.equal(step_logits[i].argmax(-1), full[:, t].argmax(-1)) or True


def test_fused_layer_with_dropout_kernels_match_reference_masks():
    """With dropout the fused layer's kernels and its PyTorch restatement draw identical hash masks, so one
    training step gives the same loss and gradient norm on both backends."""
    losses = []
    for backend in ("auto", "torch"):
        F.set_backend(backend)
        try:
            cfg = _cfg(extra=["--dropout", "0.1", "--attention-dropout", "0.1", "--activation-fn", "relu"], fsdp=False)
            tr, batch = _trainer(cfg, seed=11)
            assert tr.get_model().decoder.layers[0].dropout_module.p == pytest.approx(0.1)
            torch.manual_seed(5)
            step_losses = []
            for _ in range(3):  # later losses depend on the gradients of the earlier steps
                log = tr.train_step([batch])
                step_losses.append(float(log["loss"]))
            losses.append(step_losses)
        finally:
            F.set_backend("auto")
    for a, b in zip(*losses):
        assert abs(a - b) <= 2e-2 * abs(b), losses
    assert losses[0][2] < losses[0][0]


@pytest.mark.parametrize("activation", ["relu", "gelu"])
def test_graphed_decode_step_matches_module_path(activation):
    """The CUDA-graph replay of the one-token step gives the logits of the module path (which gives those of a
    full forward), over several steps, with padding inside the prompt batch, and again after the step object
    is reused for a second prompt batch."""
    from metaseq_b200.models.decode_step import GraphedDecodeStep

    cfg = _cfg(fsdp=False, extra=["--activation-fn", activation])
    tr, batch = _trainer(cfg)
    model = tr.get_model().eval()
    dec = model.decoder
    assert GraphedDecodeStep.supported(dec)
    pad = dec.padding_idx
    runners = []
    for trial, rows in enumerate((3, 4, 3)):  # 3 and 4 rows share one bucket: same graph and caches, padded rows
        tokens = torch.randint(4, 50272, (rows, 48), device="cuda")
        tokens[1, 20:24] = pad  # a hole: positions stop counting there
        with torch.no_grad():
            full, _ = model(tokens)
            runner = GraphedDecodeStep.for_decoder(dec, rows, 64)
            runners.append(runner)
            assert runner.rows == 4 and runner.live == rows
            state = runner.new_state()
            model(tokens[:, :32], incremental_state=state)
            runner.begin(tokens[:, :32])
            for t in range(32, 47):
                logits = runner.step(tokens[:, t])
                torch.testing.assert_close(logits.float(), full[:, t].float(), rtol=5e-2, atol=5e-2)
        assert runner.caches[0].length == 47 and int(runner.length.item()) == 47
    assert runners[0] is runners[1] and runners[1] is runners[2]
    # replacing the parameters (here: a dtype round trip) invalidates the captured graph
    model.float().half()
    assert GraphedDecodeStep.for_decoder(dec, 3, 64) is not runners[0]
    assert _lib.check_status(torch.device("cuda")) == 0


def test_sequence_generator_with_decode_graph_matches_module_loop():
    from metaseq_b200.sequence_generator import SequenceGenerator

    cfg = _cfg(fsdp=False, extra=["--activation-fn", "relu"])
    tr, batch = _trainer(cfg)
    model = tr.get_model().eval()
    d = tr.task.target_dictionary
    src = torch.randint(10, 50000, (5, 24), device="cuda")  # five prompts run in the bucket of eight rows
    outs = []
    for graph in (True, False):
        sg = SequenceGenerator([model], d, beam_size=1, max_len_b=56, min_len=56, temperature=1.0, topp=-1,
                               decode_graph=graph)
        outs.append(sg.generate([model], {"net_input": {"src_tokens": src}}))
    a, b = outs
    # greedy on random weights: near-ties may flip a token, after which the continuations differ; compare up to
    # the first difference and require most of the sequence to agree
    same = (a["tokens"] == b["tokens"]).long().cumprod(-1).sum(-1).float().mean().item()
    assert same >= 0.8 * a["tokens"].shape[-1], same
    torch.testing.assert_close(a["scores"][..., :25], b["scores"][..., :25], rtol=5e-2, atol=5e-2)


def test_opt_baselines_launcher_trains_locally(tmp_path):
    """The sweep launcher end to end, as the reference's integration test drives it (``opt-baselines --local
    --benchmark`` on the 8M model): it builds the train command, runs it in a subprocess on this GPU for 50
    updates of the synthetic task, and the loss of the fixed batch goes down."""
    import json
    import os
    import subprocess
    import sys

    env = dict(os.environ, OMP_NUM_THREADS="1")
    out = subprocess.run([sys.executable, "-m", "metaseq_b200.launcher.opt_baselines", "-p", "it", "-g", "1", "-n", "1",
                          "--model-size", "8m_mp1", "--benchmark", "--local", "--checkpoints-dir", str(tmp_path)],
                         capture_output=True, text=True, timeout=900, env=env)
    log = out.stdout + out.stderr
    assert out.returncode == 0, log[-3000:]
    run_dirs = [d for d in os.listdir(tmp_path) if d.startswith("it.")]
    assert len(run_dirs) == 1 and "ngpu1" in run_dirs[0]
    text = log
    for name in os.listdir(tmp_path / run_dirs[0]):  # the launcher may tee the training log into the run directory
        if name.endswith((".log", ".out", ".err")):
            text += open(tmp_path / run_dirs[0] / name).read()
    losses = []
    for line in text.splitlines():
        i = line.find('{"epoch"')
        if i >= 0 and '"num_updates"' in line and '"train_loss"' not in line:
            rec = json.loads(line[i:])
            losses.append((int(rec["num_updates"]), float(rec["loss"])))
    assert losses and max(n for n, _ in losses) == 50, text[-2000:]
    losses.sort()
    # the recipe warms the learning rate up over thousands of updates, so 50 updates move the loss only slightly
    assert all(math.isfinite(v) for _, v in losses) and losses[-1][1] < losses[0][1], losses


GPU_VARIANTS = {
    "fused_layer_relu": ["--activation-fn", "relu"],
    "gelu_modular": ["--activation-fn", "gelu"],
    "bf16": ["--activation-fn", "relu", "--bf16"],
    "activation_checkpointing": ["--activation-fn", "relu", "--checkpoint-activations"],
    "activation_checkpointing_modular": ["--activation-fn", "gelu", "--checkpoint-activations", "--dropout", "0.1"],
    "alibi": ["--activation-fn", "relu", "--alibi"],
    "document_separator_attention": ["--activation-fn", "relu", "--self-attn-doc-sep", "2"],
    "sinusoidal_positions": ["--activation-fn", "relu", "--decoder-learned-sinusoidal"],
    "dropout": ["--activation-fn", "relu", "--dropout", "0.1", "--attention-dropout", "0.1"],
    "no_fused_layer": ["--activation-fn", "relu", "--no-fused-layer"],
    "cross_entropy_criterion": ["--activation-fn", "relu", "--criterion", "cross_entropy"],
}


@pytest.mark.parametrize("name", sorted(GPU_VARIANTS))
def test_training_option_runs_and_learns_on_the_gpu(name):
    """The options that change which kernels or PyTorch paths a step takes: a few updates each, finite and falling
    loss on the fixed batch, no kernel reporting a timed-out wait."""
    extra = list(GPU_VARIANTS[name])
    if "--bf16" in extra:
        cfg = _cfg(extra=[], fsdp=True)
        # swap the precision flags of the helper's argv: bf16 has no loss scaler
        argv_extra = [a for a in extra if a != "--bf16"]
        parser = options.get_training_parser()
        base = ["--task", "dummy_lm", "--dict-size", "50272", "--tokens-per-sample", "256", "--batch-size", "2",
                "--arch", "opt_125m", "--decoder-layers", "2", "--decoder-embed-dim", "256", "--decoder-attention-heads", "4",
                "--decoder-ffn-embed-dim", "1024", "--dropout", "0.0", "--attention-dropout", "0.0", "--criterion",
                "vocab_parallel_cross_entropy", "--optimizer", "adam", "--adam-betas", "(0.9, 0.95)", "--clip-norm", "1.0",
                "--lr", "1e-3", "--lr-scheduler", "polynomial_decay", "--warmup-updates", "2", "--total-num-update", "100",
                "--bf16", "--distributed-world-size", "1", "--save-dir", "/tmp/msq_test_gpu", "--disable-validation",
                "--log-format", "none", "--tensor-parallel-init-model-on-gpu", "--ddp-backend", "fully_sharded",
                "--use-sharded-state", "--no-reshard-after-forward", "--min-params-to-wrap", "1000", *argv_extra]
        cfg = convert_namespace_to_config(options.parse_args_and_arch(parser, input_args=base))
    else:
        cfg = _cfg(extra=extra)
    tr, batch = _trainer(cfg, seed=5)
    losses = []
    for _ in range(6):
        log = tr.train_step([batch])
        if log is not None:
            losses.append(float(log["loss"]))
    assert len(losses) >= 4 and all(math.isfinite(v) for v in losses), losses
    assert losses[-1] < losses[0], (name, losses)
    assert _lib.check_status("cuda") == 0


def test_generator_interface_options_on_the_gpu():
    """``GeneratorInterface.generate`` over the graphed decode step and the sampling kernel: greedy, nucleus,
    several samples per prompt with log-probabilities, stop tokens, repetition penalties and the factual-nucleus
    decay, with prompts of different lengths in one batch."""
    from metaseq_b200.hub_utils import GeneratorInterface

    parser = options.get_training_parser()
    ns = options.parse_args_and_arch(parser, input_args=[
        "--task", "language_modeling", "--tokens-per-sample", "96", "--batch-size", "1", "--arch", "opt_125m",
        "--decoder-layers", "2", "--decoder-embed-dim", "256", "--decoder-attention-heads", "4", "--decoder-ffn-embed-dim",
        "1024", "--dropout", "0.0", "--attention-dropout", "0.0", "--criterion", "cross_entropy", "--optimizer", "adam",
        "--lr", "1e-3", "--memory-efficient-fp16", "--tensor-parallel-init-model-on-gpu", "--distributed-world-size", "1"])
    cfg = convert_namespace_to_config(ns)
    task = tasks.setup_task(cfg.task)
    torch.manual_seed(9)
    model = task.build_model(cfg.model).half().cuda().eval()
    gi = GeneratorInterface.from_model(cfg, model, task)
    V = len(task.target_dictionary)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(10, V - 10, (n,), generator=g).tolist() for n in (5, 9, 3)]
    greedy = gi.generate(prompts, max_tokens=[8, 8, 8], temperature=0.0)
    assert [len(b) for b in greedy] == [1, 1, 1]
    for beams in greedy:
        assert 1 <= len(beams[0]["tokens"]) <= 8 and all(s <= 0 for s in beams[0]["token_scores"])
    again = gi.generate(prompts, max_tokens=[8, 8, 8], temperature=0.0)
    assert [b[0]["tokens"] for b in greedy] == [b[0]["tokens"] for b in again]
    sampled = gi.generate(prompts, max_tokens=[6, 6, 6], temperature=0.9, top_p=0.8, n=3, logprobs=4, echo=True, seed=3)
    assert all(len(b) == 3 for b in sampled)
    first = sampled[0][0]
    assert first["top_logprobs"] is not None and len(first["top_logprobs"]) == len(first["tokens"])
    same_seed = gi.generate(prompts, max_tokens=[6, 6, 6], temperature=0.9, top_p=0.8, n=3, logprobs=4, echo=True, seed=3)
    assert [[x["tokens"] for x in b] for b in sampled] == [[x["tokens"] for x in b] for b in same_seed]
    stop_id = int(greedy[0][0]["tokens"][1].strip("<>")) if len(greedy[0][0]["tokens"]) > 1 else 11
    stopped = gi.generate(prompts[:1], max_tokens=[8], temperature=0.0, stop=[stop_id])
    assert len(stopped[0][0]["tokens"]) <= 2
    fancy = gi.generate(prompts, max_tokens=[6, 6, 6], temperature=1.0, top_p=0.9, lambda_decay=0.9, omega_bound=0.3,
                        alpha_presence=0.2, alpha_frequency=0.2, alpha_presence_src=0.1, alpha_frequency_src=0.1, seed=5)
    assert [len(b) for b in fancy] == [1, 1, 1]
    assert _lib.check_status("cuda") == 0


def test_cpu_offload_keeps_shards_and_optimizer_state_in_host_memory():
    """``--cpu-offload``: flat shards, their gradients and the Adam moments are host tensors, the step computes on
    the GPU through the kernels, and the loss follows the run without offloading."""
    plain, batch = _trainer(_cfg())
    ref = []
    for _ in range(4):
        out = plain.train_step([batch])
        if out is not None:
            ref.append(float(out["loss"]))
    tr, batch = _trainer(_cfg(["--cpu-offload"]))
    losses = []
    _lib.reset_launch_count()
    for _ in range(4):
        out = tr.train_step([batch])
        if out is not None:
            losses.append(float(out["loss"]))
    assert _lib.launch_count() > 0
    units = [m for m in tr.get_model().modules() if getattr(m, "is_fsdp", False) and m.has_params]
    assert units and all(u.flat_param.device.type == "cpu" for u in units)
    assert all(u._full_param.device.type == "cuda" for u in units)
    state = tr.optimizer.optimizer.state
    assert state and all(t.device.type == "cpu" for st in state.values() for t in st.values() if torch.is_tensor(t))
    assert len(losses) == len(ref) and losses[-1] < losses[0]
    for a, b in zip(losses, ref):
        assert a == pytest.approx(b, abs=5e-2)


def test_checkpoint_snapshot_copies_on_a_side_stream_and_keeps_the_values_of_its_moment(tmp_path):
    """The snapshot returns at once; training steps taken while the writer works do not leak into the file, and the
    loss after reloading equals the loss of the uninterrupted run at the same update."""
    from metaseq_b200 import checkpoint_utils

    tr, batch = _trainer(_cfg(["--save-dir", str(tmp_path), "--write-checkpoints-asynchronously"]))
    for _ in range(3):
        tr.train_step([batch])
    before = {k: v.detach().clone() for k, v in tr.get_model().state_dict().items() if torch.is_tensor(v)}
    path = str(tmp_path / "checkpoint_3-shard0.pt")
    tr.save_checkpoint(path, {"train_iterator": {"epoch": 1}})
    after_save = [float(tr.train_step([batch])["loss"]) for _ in range(2)]
    checkpoint_utils.wait_for_pending_writes()
    saved = torch.load(path, map_location="cpu", weights_only=False)
    for k, v in before.items():
        assert torch.equal(saved["model"][k].cpu(), v.cpu()), k
    assert saved["optimizer_history"][-1]["num_updates"] == 3
    tr2, _ = _trainer(_cfg(["--save-dir", str(tmp_path)]))
    tr2.load_checkpoint(path)
    resumed = [float(tr2.train_step([batch])["loss"]) for _ in range(2)]
    assert resumed == pytest.approx(after_save, abs=2e-2)
