"""Infrastructure pieces the reference tests with mocks: the post-checkpoint callback (fake NFS directory, fake
azcopy), the object collectives over CPU ranks, and activation checkpointing against plain autograd."""
import datetime
import os
import socket
import types

import pytest
import torch

from metaseq_b200 import checkpoint_utils
from metaseq_b200.cli import train as train_cli


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ------------------------------------------------------- post-checkpoint callback
def _ckpt_cfg(upload, world=1):
    ck = types.SimpleNamespace(cloud_upload_path=upload, nfs_eval_script_path=None, nfs_eval_frequency=1,
                               nfs_eval_num_attempts=1, nfs_eval_attempt_wait_minutes=0)
    return types.SimpleNamespace(checkpoint=ck, distributed_training=types.SimpleNamespace(distributed_world_size=world))


def test_checkpoint_callback_copies_to_nfs_atomically_and_removes_the_local_file(tmp_path):
    local = tmp_path / "local"
    nfs = tmp_path / "nfs"
    local.mkdir()
    nfs.mkdir()
    f = local / "checkpoint_18-model_part-0-shard0.pt"
    f.write_bytes(b"weights")
    last = local / "checkpoint_last-model_part-0-shard0.pt"
    train_cli.post_checkpoint_callback(_ckpt_cfg(f"nfs:{nfs}"), 18, False, str(f), [str(last)])
    # one directory per checkpoint; the step leaves the file name, so <dir>/checkpoint.pt is the loader's prefix
    target = nfs / "checkpoint_18" / "checkpoint-model_part-0-shard0.pt"
    assert target.read_bytes() == b"weights" and not f.exists()
    assert [p.name for p in (nfs / "checkpoint_18").iterdir()] == [target.name]  # no temporary file left behind
    alias = nfs / "checkpoint_last" / last.name
    assert os.path.islink(alias) and alias.read_bytes() == b"weights"
    assert train_cli._checkpoint_add_directory("checkpoint3.pt") == ("checkpoint3", "checkpoint.pt")
    with pytest.raises(AssertionError):
        train_cli._checkpoint_add_directory("model.pt")


def test_nfs_evaluation_waits_for_all_parts_then_runs_the_script(tmp_path, monkeypatch, caplog):
    nfs = tmp_path / "nfs"
    (nfs / "checkpoint_20").mkdir(parents=True)
    (nfs / "checkpoint_20" / "checkpoint-shard0.pt").write_bytes(b"a")
    (nfs / "checkpoint_20" / "_checkpoint-shard1.pt").write_bytes(b"b")  # still being copied
    script = tmp_path / "eval.sh"
    out = tmp_path / "seen.txt"
    script.write_text(f'echo "$1" > {out}\n')
    monkeypatch.setenv("METASEQ_SAVE_DIR", str(tmp_path))
    cfg = _ckpt_cfg(f"nfs:{nfs}", world=2)
    cfg.checkpoint.nfs_eval_script_path = "eval.sh"
    cfg.checkpoint.nfs_eval_frequency = 10
    cfg.checkpoint.nfs_eval_num_attempts = 2
    with caplog.at_level("ERROR"):
        train_cli.nfs_evaluation(cfg, 20, False, "checkpoint_20", str(nfs))
    assert not out.exists() and "only 1/2 checkpoint parts" in caplog.text
    os.replace(nfs / "checkpoint_20" / "_checkpoint-shard1.pt", nfs / "checkpoint_20" / "checkpoint-shard1.pt")
    train_cli.nfs_evaluation(cfg, 25, False, "checkpoint_20", str(nfs))  # not a multiple of the frequency
    assert not out.exists()
    train_cli.nfs_evaluation(cfg, 25, True, "checkpoint_20", str(nfs))  # the final checkpoint is always evaluated
    assert out.read_text().strip() == str(nfs / "checkpoint_20" / "checkpoint.pt")
    out.unlink()
    train_cli.nfs_evaluation(cfg, 20, False, "checkpoint_20", str(nfs))
    assert out.exists()


def test_checkpoint_callback_uploads_with_azcopy_and_fails_loudly(tmp_path, monkeypatch):
    f = tmp_path / "checkpoint_6-model_part-0-shard0.pt"
    f.write_bytes(b"w")
    last = tmp_path / "checkpoint_last-model_part-0-shard0.pt"
    calls = []

    def fake_azcopy(cmd, stdout):
        calls.append(cmd)
        return types.SimpleNamespace(returncode=0, stdout=b"")

    monkeypatch.setattr(train_cli, "_run_azcopy", fake_azcopy)
    url = "https://acct.blob.core.windows.net/container/run?sas"
    dest = f"https://acct.blob.core.windows.net/container/run/{f.name}?sas"  # the name goes before the token
    train_cli.post_checkpoint_callback(_ckpt_cfg(url), 6, False, str(f), [str(last)])
    assert calls[0][:2] == ["azcopy", "copy"] and calls[0][-2:] == [str(f), dest] and not f.exists()
    # blob storage has no symlinks: the alias is a second server-side copy
    assert calls[1][-2:] == [dest, f"https://acct.blob.core.windows.net/container/run/{last.name}?sas"]
    assert any(p.name.startswith(f.name + "_azcopy_logs_") for p in tmp_path.iterdir())
    f.write_bytes(b"w")
    monkeypatch.setattr(train_cli, "_run_azcopy", lambda cmd, stdout: types.SimpleNamespace(returncode=3, stdout=b"boom"))
    with pytest.raises(SystemExit):
        train_cli.post_checkpoint_callback(_ckpt_cfg(url), 6, False, str(f), None)


def test_checkpoint_callback_copies_to_a_plain_directory_with_aliases_as_full_copies(tmp_path):
    f = tmp_path / "checkpoint_6.pt"
    f.write_bytes(b"w")
    up = tmp_path / "up"
    up.mkdir()
    train_cli.post_checkpoint_callback(_ckpt_cfg(str(up)), 6, False, str(f), [str(tmp_path / "checkpoint_last.pt")])
    assert (up / "checkpoint_6.pt").read_bytes() == b"w" and (up / "checkpoint_last.pt").read_bytes() == b"w"
    assert not os.path.islink(up / "checkpoint_last.pt")


def test_checkpoint_callback_without_upload_recreates_symlinks(tmp_path):
    f = tmp_path / "checkpoint_6.pt"
    f.write_bytes(b"w")
    last = tmp_path / "checkpoint_last.pt"
    last.write_bytes(b"old")
    train_cli.post_checkpoint_callback(_ckpt_cfg(None), 6, False, str(f), [str(last)])
    assert os.path.islink(last) and os.readlink(last) == "checkpoint_6.pt" and last.read_bytes() == b"w"


def test_checkpoint_last_follows_mid_epoch_saves_after_an_epoch_boundary(tmp_path):
    """An end-of-epoch save, then a mid-epoch save: ``checkpoint_last`` must point at the newer state, so that a
    restart does not fall back to the epoch boundary."""
    from metaseq_b200 import checkpoint_utils

    written = []

    class FakeTrainer:
        data_parallel_rank = 0
        should_save_checkpoint_on_current_rank = True
        checkpoint_suffix = ""
        updates = 0

        def consolidate_optimizer(self):
            pass

        def get_num_updates(self):
            return self.updates

        def save_checkpoint(self, filename, extra_state, training_finished=False, async_callback_fn=None,
                            files_to_symlink_to=None):
            written.append((os.path.basename(filename), [os.path.basename(f) for f in files_to_symlink_to or []]))

    def itr(epoch, end):
        return types.SimpleNamespace(epoch=epoch, end_of_epoch=lambda: end, state_dict=lambda: {"epoch": epoch})

    ck = types.SimpleNamespace(save_dir=str(tmp_path), save_interval_epochs=1, save_interval_updates=5,
                               local_save_interval_updates=0, save_last_checkpoint=True, keep_last_updates=-1,
                               keep_last_epochs=-1)
    tr = FakeTrainer()
    tr.updates = 7
    checkpoint_utils.save_checkpoint(ck, tr, itr(1, True))
    tr.updates = 10
    checkpoint_utils.save_checkpoint(ck, tr, itr(2, False))
    tr.updates = 11
    checkpoint_utils.save_checkpoint(ck, tr, itr(2, False))  # not a multiple of the interval: nothing is written
    assert written == [("checkpoint1.pt", ["checkpoint_last.pt"]), ("checkpoint_10.pt", ["checkpoint_last.pt"])]
    ck.save_last_checkpoint = False
    tr.updates = 12
    checkpoint_utils.save_checkpoint(ck, tr, itr(2, False), training_finished=True)
    assert len(written) == 2


# --------------------------------------------------------------- object collectives
def _collective_rank(rank, world, port, out):
    import torch.distributed as dist

    from metaseq_b200.parallel import utils as du

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    obj = {"rank": rank, "list": list(range(rank + 1)), "tensor": torch.arange(3) + rank, "text": "x" * (10 * rank)}
    gathered = du.all_gather_list(obj, group=None, max_size=4096)
    payload = {"a": torch.arange(6).view(2, 3).float(), "nested": [1, {"b": torch.ones(2)}], "s": "hello"} if rank == 0 else None
    received = du.broadcast_object(payload, src_rank=0, group=None, dist_device=torch.device("cpu"))
    stats = du.all_reduce_dict({"loss": float(rank + 1), "n": 2.0}, device=torch.device("cpu"), group=None)
    out[rank] = dict(ranks=[g["rank"] for g in gathered], lens=[len(g["list"]) for g in gathered],
                     tensors=[g["tensor"].tolist() for g in gathered], texts=[len(g["text"]) for g in gathered],
                     bcast=(received["a"].tolist(), received["nested"][1]["b"].tolist(), received["s"]),
                     stats={k: float(v) for k, v in stats.items()})
    dist.destroy_process_group()


def test_object_collectives_over_cpu_ranks():
    import torch.multiprocessing as mp

    world = 3
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_collective_rank, args=(world, _free_port(), out), nprocs=world, join=True)
        res = dict(out)
    for r in range(world):
        assert res[r]["ranks"] == [0, 1, 2] and res[r]["lens"] == [1, 2, 3] and res[r]["texts"] == [0, 10, 20]
        assert res[r]["tensors"] == [[0, 1, 2], [1, 2, 3], [2, 3, 4]]
        assert res[r]["bcast"] == ([[0.0, 1.0, 2.0], [3.0, 4.0, 5.0]], [1.0, 1.0], "hello")
        assert res[r]["stats"] == {"loss": 6.0, "n": 6.0}


# ------------------------------------------------------------ activation checkpointing
class _Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a = torch.nn.Linear(16, 32)
        self.drop = torch.nn.Dropout(0.3)  # the recomputation must replay the same mask
        self.b = torch.nn.Linear(32, 16)

    def forward(self, x):
        return x + self.b(self.drop(torch.relu(self.a(x))))


@pytest.mark.parametrize("offload", [False, True])
def test_activation_checkpointing_matches_plain_autograd_with_dropout(offload):
    from metaseq_b200.modules.checkpoint_activations import checkpoint_wrapper

    def run(wrap):
        torch.manual_seed(0)
        net = torch.nn.Sequential(_Block(), _Block(), _Block())
        if wrap:
            for i in range(len(net)):
                net[i] = checkpoint_wrapper(net[i], offload_to_cpu=offload)
        net.train()
        x = torch.randn(5, 16, generator=torch.Generator().manual_seed(1), requires_grad=True)
        torch.manual_seed(7)  # dropout stream
        loss = net(x).pow(2).sum()
        loss.backward()
        gnorm = torch.sqrt(sum(p.grad.pow(2).sum() for p in net.parameters()))
        return float(loss.detach()), float(gnorm), x.grad.clone()

    plain, ckpt = run(False), run(True)
    assert plain[0] == pytest.approx(ckpt[0], rel=1e-6) and plain[1] == pytest.approx(ckpt[1], rel=1e-5)
    assert torch.allclose(plain[2], ckpt[2], atol=1e-6)


def test_checkpointing_state_queries_and_disable_context():
    import torch

    from metaseq_b200.modules import checkpoint_activations as ca

    class Probe(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(4, 4)
            self.seen = []

        def forward(self, x):
            self.seen.append((ca.is_checkpointing(), ca.is_recomputing()))
            return self.lin(x).relu()

    torch.manual_seed(0)
    m = ca.checkpoint_wrapper(Probe())
    x = torch.randn(3, 4, requires_grad=True)
    m(x).sum().backward()
    assert m.seen == [(True, False), (False, True)]  # dropped pass, then the recomputation
    grad = x.grad.clone()
    assert not ca.is_checkpointing() and not ca.is_recomputing() and not ca.is_checkpointing_disabled()
    m.seen.clear()
    x.grad = None
    with ca.disable_checkpointing():
        assert ca.is_checkpointing_disabled()
        m(x).sum().backward()
    assert m.seen == [(False, False)]  # one ordinary pass
    assert torch.allclose(x.grad, grad)


def test_loss_spike_guard_keeps_spikes_out_of_the_running_mean():
    """With a threshold, a spike returns its ratio and leaves the mean alone; ordinary steps move the mean by
    alpha = 0.2; without a threshold the mean follows every step."""
    from metaseq_b200.trainer import Trainer

    t = types.SimpleNamespace(_ewm_loss=None, _skipped_loss_spikes=0, _spike_guard_on=Trainer._spike_guard_on)
    assert Trainer.skip_spike(t, 10.0, 1.5) == 1.0 and t._ewm_loss == 10.0
    assert Trainer.skip_spike(t, 11.0, 1.5) == pytest.approx(1.1)
    assert t._ewm_loss == pytest.approx(10.2)
    assert Trainer.skip_spike(t, 30.0, 1.5) == pytest.approx(30.0 / 10.2)
    assert t._ewm_loss == pytest.approx(10.2) and t._skipped_loss_spikes == 1
    off = types.SimpleNamespace(_ewm_loss=None, _skipped_loss_spikes=0, _spike_guard_on=Trainer._spike_guard_on)
    Trainer.skip_spike(off, 10.0, -1)
    Trainer.skip_spike(off, 30.0, -1)
    assert off._ewm_loss == pytest.approx(14.0) and off._skipped_loss_spikes == 0


def test_host_snapshot_is_a_private_copy_and_the_writer_waits_for_it(tmp_path):
    from metaseq_b200 import checkpoint_utils

    snap = checkpoint_utils.HostSnapshot()
    live = {"model": {"w": torch.arange(6.0), "half": torch.ones(3, dtype=torch.float16)}, "n": 3, "name": "x"}
    state = snap.take(live, cast_to_fp32=True)
    live["model"]["w"].add_(100)  # training goes on while the writer serialises
    assert state["model"]["w"].tolist() == [0.0, 1.0, 2.0, 3.0, 4.0, 5.0] and state["n"] == 3 and state["name"] == "x"
    assert state["model"]["half"].dtype == torch.float32
    called = []
    path = str(tmp_path / "ckpt.pt")
    checkpoint_utils.write_checkpoint(state, path, asynchronous=True, ready=lambda: called.append(1))
    checkpoint_utils.wait_for_pending_writes()
    assert called == [1]
    assert torch.load(path, weights_only=False)["model"]["w"].tolist() == [0.0, 1.0, 2.0, 3.0, 4.0, 5.0]


def test_resume_from_shared_directory_takes_the_newest_complete_checkpoint(tmp_path, monkeypatch):
    """With ``--cloud-upload-path nfs:<dir>`` a restart looks in that directory, not in the local save directory:
    the newest ``checkpoint_N`` with one finished file per rank wins; unfinished copies do not count."""
    nfs = tmp_path / "nfs"
    for step, names in ((10, ["checkpoint-shard0.pt", "checkpoint-shard1.pt"]),
                        (20, ["checkpoint-shard0.pt", "_checkpoint-shard1.pt"])):
        d = nfs / f"checkpoint_{step}"
        d.mkdir(parents=True)
        for n in names:
            (d / n).write_bytes(b"x")
    (nfs / "checkpoint_last").mkdir()
    seen = {}

    class FakeTrainer:
        checkpoint_suffix = "-shard0"

        def load_checkpoint(self, path, *a, **k):
            seen["path"] = path
            return None

        def get_train_iterator(self, epoch, **k):
            return types.SimpleNamespace(epoch=epoch)

        def lr_step(self, epoch):
            pass

    ck = types.SimpleNamespace(
        reset_optimizer=False, reset_lr_scheduler=False, optimizer_overrides="{}", reset_meters=False,
        reset_dataloader=False, finetune_from_model=None, restore_file="checkpoint_last.pt",
        save_dir=str(tmp_path / "local"), cloud_upload_path=f"nfs:{nfs}")
    cfg = types.SimpleNamespace(checkpoint=ck)
    monkeypatch.setattr(checkpoint_utils.dist_utils, "get_global_world_size", lambda: 2)
    checkpoint_utils.load_checkpoint(cfg, FakeTrainer())
    assert seen["path"] == str(nfs / "checkpoint_10" / "checkpoint-shard0.pt")
    ck.restore_file = str(nfs / "checkpoint_20" / "checkpoint.pt")  # an explicit file is taken as given
    checkpoint_utils.load_checkpoint(cfg, FakeTrainer())
    assert seen["path"] == str(nfs / "checkpoint_20" / "checkpoint-shard0.pt")
    monkeypatch.setenv("SLURM_RESTART_COUNT", "1")  # ... unless the job was requeued
    checkpoint_utils.load_checkpoint(cfg, FakeTrainer())
    assert seen["path"] == str(nfs / "checkpoint_10" / "checkpoint-shard0.pt")


# ------------------------------------------------- column-parallel product with overlapped backward collectives
def _async_linear_rank(rank, world, port, out):
    import torch.distributed as dist

    from metaseq_b200.parallel import mpu
    from metaseq_b200.parallel.layers import LinearWithGradAccumulationAndAsyncCommunication as AsyncLinear

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    mpu.initialize_model_parallel(world)
    torch.manual_seed(0)
    T, B, K, N = 4 * world, 2, 6, 8 * world
    x_full = torch.randn(T, B, K, dtype=torch.double)
    w_full = torch.randn(N, K, dtype=torch.double)
    b_full = torch.randn(N, dtype=torch.double)
    g_full = torch.randn(T, B, N, dtype=torch.double)
    n = N // world
    w = w_full[rank * n:(rank + 1) * n].clone().requires_grad_()
    b = b_full[rank * n:(rank + 1) * n].clone().requires_grad_()
    g = g_full[..., rank * n:(rank + 1) * n]
    res = {}
    # plain tensor parallelism: the input is replicated, its gradient is all-reduced behind the weight gradient
    x = x_full.clone().requires_grad_()
    y = AsyncLinear.apply(x, w, b, False, True, False)
    y.backward(g)
    res["tp"] = (y.detach(), x.grad.clone(), w.grad.clone(), b.grad.clone())
    # sequence parallelism: rows are gathered going in, the input gradient is reduce-scattered; the weight
    # gradient goes straight into main_grad
    w.grad = b.grad = None
    w.main_grad = torch.zeros(n, K)
    t = T // world
    xs = x_full[rank * t:(rank + 1) * t].clone().requires_grad_()
    y = AsyncLinear.apply(xs, w, b, True, False, True)
    y.backward(g)
    res["sp"] = (y.detach(), xs.grad.clone(), w.main_grad.clone(), w.grad, b.grad.clone())
    out[rank] = res
    mpu.destroy_model_parallel()
    dist.destroy_process_group()


def test_column_parallel_product_with_async_communication_matches_the_full_product():
    import torch.multiprocessing as mp

    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_async_linear_rank, args=(world, _free_port(), out), nprocs=world, join=True)
        res = dict(out)
    torch.manual_seed(0)
    T, B, K, N = 4 * world, 2, 6, 8 * world
    x = torch.randn(T, B, K, dtype=torch.double, requires_grad=True)
    w = torch.randn(N, K, dtype=torch.double, requires_grad=True)
    b = torch.randn(N, dtype=torch.double, requires_grad=True)
    g = torch.randn(T, B, N, dtype=torch.double)
    y = torch.nn.functional.linear(x, w, b)
    y.backward(g)
    n, t = N // world, T // world
    for r in range(world):
        cols = slice(r * n, (r + 1) * n)
        y_r, dx_r, dw_r, db_r = res[r]["tp"]
        assert torch.allclose(y_r, y.detach()[..., cols]) and torch.allclose(dx_r, x.grad)
        assert torch.allclose(dw_r, w.grad[cols]) and torch.allclose(db_r, b.grad[cols])
        y_r, dx_r, main_grad, dw_r, db_r = res[r]["sp"]
        assert torch.allclose(y_r, y.detach()[..., cols]) and torch.allclose(dx_r, x.grad[r * t:(r + 1) * t])
        assert dw_r is None and torch.allclose(main_grad.double(), w.grad[cols], atol=1e-5)
        assert torch.allclose(db_r, b.grad[cols])


def test_restart_fetches_the_newest_checkpoint_of_this_rank_from_blob_storage(tmp_path, monkeypatch):
    calls, seen = [], {}
    listing = (b"INFO: checkpoint_10-model_part-0-shard0.pt;  Content Length: 1.00 GiB\n"
               b"INFO: checkpoint_20-model_part-0-shard0.pt;  Content Length: 1.00 GiB\n"
               b"INFO: checkpoint_30-model_part-0-shard1.pt;  Content Length: 1.00 GiB\n"
               b"INFO: checkpoint_last-model_part-0-shard0.pt;  Content Length: 1.00 GiB\n")

    def fake_azcopy(args):
        calls.append(args)
        if args[0] == "copy":
            open(args[2], "wb").write(b"ckpt")
        return types.SimpleNamespace(returncode=0, stdout=listing if args[0] == "list" else b"", stderr=b"")

    monkeypatch.setattr(checkpoint_utils, "_run_azcopy", fake_azcopy)

    class FakeTrainer:
        checkpoint_suffix = "-model_part-0-shard0"

        def load_checkpoint(self, path, *a, **k):
            seen["path"] = path
            return None

        def get_train_iterator(self, epoch, **k):
            return types.SimpleNamespace(epoch=epoch)

        def lr_step(self, epoch):
            pass

    url = "https://acct.blob.core.windows.net/cont/run?sig=abc"
    ck = types.SimpleNamespace(
        reset_optimizer=False, reset_lr_scheduler=False, optimizer_overrides="{}", reset_meters=False,
        reset_dataloader=False, finetune_from_model=None, restore_file="checkpoint_last.pt",
        save_dir=str(tmp_path / "local"), cloud_upload_path=url)
    checkpoint_utils.load_checkpoint(types.SimpleNamespace(checkpoint=ck), FakeTrainer())
    local = str(tmp_path / "local" / "checkpoint_last-model_part-0-shard0.pt")
    assert calls[0] == ["list", url]
    assert calls[1] == ["copy", "https://acct.blob.core.windows.net/cont/run/checkpoint_20-model_part-0-shard0.pt?sig=abc", local]
    assert seen["path"] == local and open(local, "rb").read() == b"ckpt"

    # an empty container is a first launch, not an error
    listing = b""
    calls.clear()
    checkpoint_utils.load_checkpoint(types.SimpleNamespace(checkpoint=ck), FakeTrainer())
    assert [c[0] for c in calls] == ["list"]

    # without an upload path, a requeued job that began from an explicit file continues from its own last checkpoint
    ck.cloud_upload_path = None
    ck.restore_file = str(tmp_path / "pretrained" / "model.pt")
    monkeypatch.setenv("SLURM_RESTART_COUNT", "2")
    checkpoint_utils.load_checkpoint(types.SimpleNamespace(checkpoint=ck), FakeTrainer())
    assert seen["path"] == local
    os.remove(local)
    checkpoint_utils.load_checkpoint(types.SimpleNamespace(checkpoint=ck), FakeTrainer())
    assert seen["path"] == str(tmp_path / "pretrained" / "model-model_part-0-shard0.pt")


def test_task_is_set_up_inside_the_sharding_context_when_asked(monkeypatch):
    from metaseq_b200.parallel import fsdp

    seen = {}

    def fake_setup(task_cfg):
        seen["inside"] = fsdp._WRAP_KWARGS is not None
        seen["flags"] = (d.memory_efficient_fp16, d.fp32_reduce_scatter)
        return "task"

    monkeypatch.setattr(train_cli.tasks, "setup_task", fake_setup)
    d = types.SimpleNamespace(task_ddp_backend="fully_sharded", fp16=True, memory_efficient_fp16=False,
                              fp32_reduce_scatter=True, use_sharded_state=True, no_reshard_after_forward=False,
                              cpu_offload=False, bf16=False, bucket_cap_mb=25, gradient_predivide_factor=None)
    cfg = types.SimpleNamespace(distributed_training=d, task=None,
                                common=types.SimpleNamespace(fp16=True, memory_efficient_fp16=False, bf16=False))
    assert train_cli._setup_task(cfg) == "task"
    assert seen == {"inside": True, "flags": (True, False)}
    assert (d.memory_efficient_fp16, d.fp32_reduce_scatter) == (False, True)  # put back afterwards
    d.task_ddp_backend = "none"
    train_cli._setup_task(cfg)
    assert seen["inside"] is False
