"""End to end on a CPU, through the command-line entry points a user runs: train a tiny model on JSONL shards with
the streaming task, score the checkpoint with the validation CLI, then load it through ``GeneratorInterface``
(the object behind the completions service) and generate with greedy and nucleus decoding."""
import json
import os
import subprocess
import sys

import pytest
import torch

from test_task_fileio_cpu import _write_shards, _write_tokenizer


def _run(cmd, timeout=600):
    env = dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    return out.stdout + out.stderr


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    root = tmp_path_factory.mktemp("e2e")
    vocab, merges = _write_tokenizer(root)
    data = root / "data"
    _write_shards(data, n_shards=1, docs=40)
    save = root / "ckpt"
    common = ["--task", "streaming_language_modeling", "--vocab-filename", vocab, "--merges-filename", merges,
              "--tokens-per-sample", "32", "--sample-break-mode", "none"]
    log = _run([sys.executable, "-m", "metaseq_b200.cli.train", str(data), *common, "--batch-size", "4",
                "--arch", "transformer_lm_megatron", "--decoder-layers", "2", "--decoder-embed-dim", "64",
                "--decoder-ffn-embed-dim", "128", "--decoder-attention-heads", "4", "--decoder-learned-pos",
                "--share-decoder-input-output-embed", "--activation-fn", "relu", "--dropout", "0.0",
                "--attention-dropout", "0.0", "--criterion", "cross_entropy", "--optimizer", "adam", "--lr", "3e-3",
                "--lr-scheduler", "polynomial_decay", "--warmup-updates", "2", "--total-num-update", "40",
                "--max-update", "30", "--cpu", "--distributed-world-size", "1", "--log-format", "json", "--log-interval",
                "5", "--save-dir", str(save), "--save-interval-updates", "30", "--disable-validation", "--seed", "1",
                "--num-workers", "0"])
    losses = [json.loads(line[line.find('{"epoch"'):])["loss"] for line in log.splitlines()
              if '{"epoch"' in line and '"loss"' in line and '"train_loss"' not in line]
    ckpts = sorted(p for p in os.listdir(save) if p.endswith(".pt"))
    return dict(root=root, data=data, save=save, common=common, losses=[float(x) for x in losses], ckpts=ckpts,
                vocab=vocab, merges=merges)


def test_training_cli_reduces_the_loss_and_writes_a_checkpoint(trained):
    assert len(trained["losses"]) >= 3 and trained["losses"][-1] < trained["losses"][0] - 0.5, trained["losses"]
    assert any(c.startswith("checkpoint_30") or c == "checkpoint_last.pt" for c in trained["ckpts"]), trained["ckpts"]


def _checkpoint(trained):
    for name in ("checkpoint_last.pt", "checkpoint_30.pt"):
        if name in trained["ckpts"]:
            return str(trained["save"] / name)
    return str(trained["save"] / trained["ckpts"][-1])


def test_validation_cli_scores_the_checkpoint(trained):
    log = _run([sys.executable, "-m", "metaseq_b200.cli.validate", str(trained["data"]), *trained["common"],
                "--path", _checkpoint(trained), "--batch-size", "4", "--valid-subset", "valid", "--cpu",
                "--distributed-world-size", "1", "--log-format", "json", "--num-workers", "0"])
    recs = [json.loads(line[line.find("{"):]) for line in log.splitlines() if '"valid_loss"' in line or '"loss"' in line]
    assert recs, log[-2000:]
    loss = float(next(v for r in recs for k, v in r.items() if k.endswith("loss")))
    assert 0.0 < loss < trained["losses"][0]  # better than the untrained model


def test_generator_interface_loads_the_checkpoint_and_generates(trained):
    from metaseq_b200 import options
    from metaseq_b200.dataclass.utils import convert_namespace_to_config
    from metaseq_b200.hub_utils import GeneratorInterface

    parser = options.get_generation_parser()
    args = options.parse_args_and_arch(parser, input_args=[
        str(trained["data"]), *trained["common"], "--path", _checkpoint(trained), "--bpe", "hf_byte_bpe",
        "--bpe-vocab", trained["vocab"], "--bpe-merges", trained["merges"], "--beam", "1", "--batch-size", "2", "--cpu",
        "--distributed-world-size", "1"])
    gi = GeneratorInterface(convert_namespace_to_config(args))
    gi.load_model()
    prompts = [gi.encode_fn("the quick brown"), gi.encode_fn("shard 0 corpus a doc")]
    out = gi.generate(prompts, max_tokens=[6, 6], temperature=0.0, echo=False)
    assert len(out) == 2 and all(len(beams) == 1 for beams in out)
    for beams in out:
        r = beams[0]
        assert 1 <= len(r["tokens"]) <= 6 and isinstance(r["text"], str) and len(r["token_scores"]) == len(r["tokens"])
        assert all(s <= 0 for s in r["token_scores"])
    again = gi.generate(prompts, max_tokens=[6, 6], temperature=0.0, echo=False)
    assert [b[0]["tokens"] for b in out] == [b[0]["tokens"] for b in again]  # greedy decoding is deterministic
    # the model has seen this corpus: its greedy continuation of a training prefix is corpus text
    assert any(w in out[0][0]["text"] for w in ("fox", "brown", "quick", "the")), out[0][0]["text"]
    sampled = gi.generate(prompts, max_tokens=[5, 5], temperature=0.8, top_p=0.9, n=2, logprobs=2, echo=True, seed=7)
    assert all(len(beams) == 2 for beams in sampled)
    r = sampled[0][0]
    assert r["top_logprobs"] is not None and r["text"].startswith("the quick brown")


def test_completions_service_answers_over_http(trained):
    """The hosted completions service in one process: model behind ``GeneratorInterface``, the batching thread, the
    HTTP handler; two concurrent requests are batched and answered in OpenAI format."""
    import json as _json
    import socket
    import threading
    import urllib.error
    import urllib.request
    from http.server import ThreadingHTTPServer

    from metaseq_b200 import options
    from metaseq_b200.cli import interactive_hosted as svc
    from metaseq_b200.dataclass.utils import convert_namespace_to_config
    from metaseq_b200.hub_utils import GeneratorInterface

    args = options.parse_args_and_arch(options.get_generation_parser(), input_args=[
        str(trained["data"]), *trained["common"], "--path", _checkpoint(trained), "--bpe", "hf_byte_bpe",
        "--bpe-vocab", trained["vocab"], "--bpe-merges", trained["merges"], "--beam", "1", "--batch-size", "2", "--cpu",
        "--distributed-world-size", "1"])
    gi = GeneratorInterface(convert_namespace_to_config(args))
    gi.load_model()
    svc.generator = gi
    stop = threading.Event()
    worker = threading.Thread(target=svc.batching_loop, kwargs=dict(timeout=50, stop_event=stop), daemon=True)
    worker.start()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = ThreadingHTTPServer(("127.0.0.1", port), svc.CompletionsHandler)
    threading.Thread(target=server.serve_forever, daemon=True).start()

    def post(body, path="/completions"):
        req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=_json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            return _json.loads(r.read())

    try:
        answers = [None, None]

        def ask(i, prompt):
            answers[i] = post({"prompt": prompt, "max_tokens": 5, "temperature": 0.0})

        threads = [threading.Thread(target=ask, args=(0, "the quick brown")),
                   threading.Thread(target=ask, args=(1, ["shard 0 corpus a", "the lazy"]))]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=180)
        assert answers[0] is not None and answers[1] is not None
        assert answers[0]["object"] == "text_completion" and len(answers[0]["choices"]) == 1
        assert len(answers[1]["choices"]) == 2  # one choice per prompt of the list
        for choice in answers[0]["choices"] + answers[1]["choices"]:
            assert isinstance(choice["text"], str) and "logprobs" in choice
        alt = post({"prompt": "the quick brown", "max_tokens": 4, "temperature": 0.7, "top_p": 0.9, "n": 2},
                   path="/v1/engines/tiny/completions")
        assert len(alt["choices"]) == 2
        with pytest.raises(urllib.error.HTTPError) as err:
            post({"max_tokens": 4})
        assert err.value.code == 400
    finally:
        stop.set()
        server.shutdown()
        server.server_close()


def test_resuming_mid_epoch_continues_the_same_data_order_and_losses(tmp_path):
    """The streaming data iterator, the optimizer and the schedule are restored from the checkpoint: a run stopped
    at update 6 and resumed reproduces the losses of an uninterrupted run (the reference's resume test:
    tests/test_streaming_language_modeling_task.py:24-157)."""
    import shutil

    vocab, merges = _write_tokenizer(tmp_path)
    data = tmp_path / "data"
    _write_shards(data, n_shards=1, docs=60)

    def run(save, max_update, extra=()):
        log = _run([sys.executable, "-m", "metaseq_b200.cli.train", str(data), "--task", "streaming_language_modeling",
                    "--vocab-filename", vocab, "--merges-filename", merges, "--tokens-per-sample", "16",
                    "--sample-break-mode", "none", "--batch-size", "2", "--arch", "transformer_lm_megatron",
                    "--decoder-layers", "1", "--decoder-embed-dim", "32", "--decoder-ffn-embed-dim", "64",
                    "--decoder-attention-heads", "2", "--decoder-learned-pos", "--share-decoder-input-output-embed",
                    "--dropout", "0.1", "--attention-dropout", "0.0", "--criterion", "cross_entropy", "--optimizer",
                    "adam", "--lr", "3e-3", "--lr-scheduler", "polynomial_decay", "--warmup-updates", "2",
                    "--total-num-update", "40", "--max-update", str(max_update), "--cpu", "--distributed-world-size",
                    "1", "--log-format", "json", "--log-interval", "1", "--save-dir", str(save),
                    "--save-interval-updates", "6", "--disable-validation", "--seed", "3", "--num-workers", "0", *extra])
        out = {}
        for line in log.splitlines():
            i = line.find('{"epoch"')
            if i >= 0 and '"num_updates"' in line and '"train_loss"' not in line:
                rec = json.loads(line[i:])
                out[int(rec["num_updates"])] = float(rec["loss"])
        return out

    straight = run(tmp_path / "a", 12)
    assert sorted(straight) == list(range(1, 13))
    resumed_dir = tmp_path / "b"
    resumed_dir.mkdir()
    for name in os.listdir(tmp_path / "a"):
        if name.startswith("checkpoint_6"):
            shutil.copy(tmp_path / "a" / name, resumed_dir / name)
    assert os.listdir(resumed_dir), os.listdir(tmp_path / "a")
    if not (resumed_dir / "checkpoint_last.pt").exists():
        first = sorted(os.listdir(resumed_dir))[0]
        os.symlink(first, resumed_dir / "checkpoint_last.pt")
    resumed = run(resumed_dir, 12)
    assert min(resumed) == 7 and max(resumed) == 12, resumed
    for n in range(7, 13):
        assert resumed[n] == pytest.approx(straight[n], abs=2e-3), (n, resumed[n], straight[n])


def test_interactive_cli_answers_a_prompt_from_stdin(trained):
    cmd = [sys.executable, "-m", "metaseq_b200.cli.interactive_cli", *trained["common"], "--path", _checkpoint(trained),
           "--bpe-vocab", trained["vocab"], "--bpe-merges", trained["merges"], "--model-parallel-size", "1",
           "--distributed-world-size", "1", "--cpu", "--batch-size", "1"]
    env = dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    out = subprocess.run(cmd, input="the quick brown\n\n", capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    answer = [line for line in out.stdout.splitlines() if line.strip() and "INFO" not in line and "|" not in line]
    assert answer, out.stdout[-2000:] + out.stderr[-1000:]


def test_profile_flag_writes_a_trace_and_a_memory_table(tmp_path):
    save = tmp_path / "prof"
    _run([sys.executable, "-m", "metaseq_b200.cli.train", "--task", "dummy_lm", "--dict-size", "60", "--tokens-per-sample",
          "16", "--batch-size", "2", "--arch", "transformer_lm_megatron", "--decoder-layers", "1", "--decoder-embed-dim",
          "32", "--decoder-ffn-embed-dim", "64", "--decoder-attention-heads", "2", "--criterion", "cross_entropy",
          "--optimizer", "adam", "--lr", "1e-3", "--max-update", "8", "--cpu", "--distributed-world-size", "1",
          "--log-format", "none", "--save-dir", str(save), "--disable-validation", "--save-interval-epochs", "0",
          "--save-interval-updates", "0", "--profile"])
    trace = save / "profiler_trace.json"
    assert trace.exists() and trace.stat().st_size > 1000
    events = json.loads(trace.read_text())
    assert "traceEvents" in events and len(events["traceEvents"]) > 10
    assert (save / "memory_usage.txt").exists()


def test_fixed_prompt_generation_benchmark_runs_from_a_checkpoint_directory(trained, tmp_path, capsys):
    """The directory layout that the released models use: ``reshard*.pt`` beside ``gpt2-vocab.json`` and
    ``gpt2-merges.txt``; everything else is inferred."""
    import shutil

    from metaseq_b200.benchmark import generation_benchmarks as gb

    shutil.copy(_checkpoint(trained), tmp_path / "reshard.pt")
    shutil.copy(trained["vocab"], tmp_path / "gpt2-vocab.json")
    shutil.copy(trained["merges"], tmp_path / "gpt2-merges.txt")
    seconds = gb.generation_statistics(str(tmp_path), prompts=["the quick brown fox"] * 8, cpu=True)
    out = capsys.readouterr().out
    assert seconds > 0 and "Total generation time" in out and "Words per second" in out


def test_checkpoints_move_to_a_shared_directory_and_a_restart_resumes_from_there(tmp_path):
    """``--cloud-upload-path nfs:<dir>``: every finished checkpoint ends up in ``<dir>/checkpoint_N/`` under a name
    without the step, the local copy goes away, and a second launch with an empty save directory continues from the
    newest complete directory instead of starting over."""
    vocab, merges = _write_tokenizer(tmp_path)
    data = tmp_path / "data"
    _write_shards(data, n_shards=1, docs=60)
    shared = tmp_path / "shared"
    shared.mkdir()

    def run(save, max_update):
        log = _run([sys.executable, "-m", "metaseq_b200.cli.train", str(data), "--task", "streaming_language_modeling",
                    "--vocab-filename", vocab, "--merges-filename", merges, "--tokens-per-sample", "16",
                    "--sample-break-mode", "none", "--batch-size", "2", "--arch", "transformer_lm_megatron",
                    "--decoder-layers", "1", "--decoder-embed-dim", "32", "--decoder-ffn-embed-dim", "64",
                    "--decoder-attention-heads", "2", "--decoder-learned-pos", "--share-decoder-input-output-embed",
                    "--dropout", "0.0", "--attention-dropout", "0.0", "--criterion", "cross_entropy", "--optimizer",
                    "adam", "--lr", "3e-3", "--lr-scheduler", "polynomial_decay", "--warmup-updates", "2",
                    "--total-num-update", "40", "--max-update", str(max_update), "--cpu", "--distributed-world-size",
                    "1", "--log-format", "json", "--log-interval", "1", "--save-dir", str(save),
                    "--save-interval-updates", "4", "--disable-validation", "--seed", "3", "--num-workers", "0",
                    "--cloud-upload-path", f"nfs:{shared}"])
        return sorted(int(json.loads(line[line.find('{"epoch"'):])["num_updates"]) for line in log.splitlines()
                      if '{"epoch"' in line and '"num_updates"' in line and '"train_loss"' not in line)

    first = run(tmp_path / "run1", 8)
    assert first == list(range(1, 9))
    dirs = sorted(p.name for p in shared.iterdir())
    assert "checkpoint_4" in dirs and "checkpoint_8" in dirs, dirs
    assert [p.name for p in (shared / "checkpoint_8").iterdir()] == ["checkpoint.pt"]
    assert not [n for n in os.listdir(tmp_path / "run1") if n.startswith("checkpoint_") and n.endswith(".pt")
                and not os.path.islink(tmp_path / "run1" / n)]

    second = run(tmp_path / "run2", 12)  # a fresh node: nothing local, everything on the shared directory
    assert second == list(range(9, 13)), second
    assert (shared / "checkpoint_12" / "checkpoint.pt").exists()


def test_training_validates_on_its_interval_and_logs_under_the_subset_name(tmp_path):
    """``--validate-interval-updates``: a validation pass over ``valid`` after every fourth update and at the end,
    each logged as one JSON line under the logger name of the subset, with loss and perplexity."""
    vocab, merges = _write_tokenizer(tmp_path)
    data = tmp_path / "data"
    _write_shards(data, n_shards=1, docs=60)
    log = _run([sys.executable, "-m", "metaseq_b200.cli.train", str(data), "--task", "streaming_language_modeling",
                "--vocab-filename", vocab, "--merges-filename", merges, "--tokens-per-sample", "16",
                "--sample-break-mode", "none", "--batch-size", "2", "--arch", "transformer_lm_megatron",
                "--decoder-layers", "1", "--decoder-embed-dim", "32", "--decoder-ffn-embed-dim", "64",
                "--decoder-attention-heads", "2", "--decoder-learned-pos", "--share-decoder-input-output-embed",
                "--dropout", "0.0", "--attention-dropout", "0.0", "--criterion", "cross_entropy", "--optimizer", "adam",
                "--lr", "3e-3", "--lr-scheduler", "polynomial_decay", "--warmup-updates", "2", "--total-num-update",
                "40", "--max-update", "8", "--cpu", "--distributed-world-size", "1", "--log-format", "json",
                "--log-interval", "1", "--save-dir", str(tmp_path / "ckpt"), "--seed", "3",
                "--num-workers", "0", "--valid-subset", "valid", "--validate-interval-updates", "4",
                "--batch-size-valid", "2"])
    valid = [json.loads(line[line.find("{"):]) for line in log.splitlines() if '"valid_loss"' in line]
    assert [int(r["valid_num_updates"]) for r in valid] == [4, 8], log[-3000:]
    assert all(float(r["valid_loss"]) > 0 and float(r["valid_ppl"]) > 1 for r in valid)
    assert float(valid[1]["valid_loss"]) < float(valid[0]["valid_loss"])
    assert any("| valid |" in line for line in log.splitlines() if '"valid_loss"' in line)
