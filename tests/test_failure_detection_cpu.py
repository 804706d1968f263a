"""Failure detection exercised on the host: a stalled loop, a rank that dies before a collective, checkpoint
directories left incomplete by an interrupted copy, a writer that fails mid-way, and the epoch / double-buffer
protocol of the decode all-reduce replayed by CPU threads.  Nothing here touches a GPU."""
import datetime
import os
import random
import socket
import threading
import time

import pytest
import torch

from metaseq_b200 import checkpoint_utils
from metaseq_b200.utils.watchdog import StepWatchdog


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ------------------------------------------------------------------ watchdog
def test_watchdog_stays_quiet_while_the_loop_beats_and_fires_when_it_stalls():
    fired = []
    wd = StepWatchdog(0.6, on_timeout=fired.append, poll_s=0.05).start()
    for _ in range(12):
        time.sleep(0.1)
        wd.beat()
    assert not fired and wd.fired is None
    time.sleep(1.2)  # the loop "hangs"
    assert len(fired) == 1 and "no heartbeat" in fired[0]
    wd.stop()


def test_watchdog_reports_pending_device_work_and_a_kernel_status_code():
    class NeverDone:
        def query(self):
            return False

    class Done:
        def query(self):
            return True

    fired = []
    wd = StepWatchdog(0.4, on_timeout=fired.append, poll_s=0.05).start()
    wd.watch_event(Done())
    for _ in range(8):
        time.sleep(0.1)
        wd.beat()
    assert not fired
    wd.watch_event(NeverDone())
    for _ in range(10):
        time.sleep(0.1)
        wd.beat()  # the host keeps stepping, the device does not finish
    assert len(fired) == 1 and "device work still pending" in fired[0]
    wd.stop()
    codes = iter([0, 0, 5, 5, 5, 5, 5, 5])
    fired2 = []
    wd2 = StepWatchdog(5.0, on_timeout=fired2.append, poll_s=0.05, status_fn=lambda: next(codes, 5)).start()
    time.sleep(0.5)
    assert len(fired2) == 1 and "status word 5" in fired2[0]
    wd2.stop()


def test_default_watchdog_action_interrupts_the_main_thread():
    wd = StepWatchdog(0.3, poll_s=0.05).start()
    with pytest.raises(KeyboardInterrupt):
        for _ in range(100):
            time.sleep(0.1)  # never beats
    assert wd.fired is not None
    wd.stop()


# ---------------------------------------------------- a rank that never joins
def _rank_main(rank, world, port, die, out):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    t = torch.ones(4)
    dist.all_reduce(t)  # everyone is alive for the first collective
    if die and rank == 1:
        os._exit(17)  # dies between steps, with nothing of its own in flight
    t0 = time.time()
    try:
        dist.all_reduce(t)
        out[rank] = ("ok", time.time() - t0)
    except Exception as e:  # noqa: BLE001
        out[rank] = ("error", time.time() - t0, type(e).__name__)


def test_surviving_ranks_get_an_error_within_the_process_group_timeout():
    import torch.multiprocessing as mp

    world = 3
    with mp.Manager() as mgr:
        out = mgr.dict()
        ctx = mp.start_processes(_rank_main, args=(world, _free_port(), True, out), nprocs=world, join=False,
                                 start_method="spawn")
        deadline = time.time() + 60
        while time.time() < deadline and any(p.is_alive() for p in ctx.processes):
            time.sleep(0.2)
        for p in ctx.processes:
            if p.is_alive():
                p.terminate()
        results = dict(out)
    assert ctx.processes[1].exitcode == 17
    for r in (0, 2):
        assert r in results and results[r][0] == "error", results
        assert results[r][1] < 30, results  # bounded by the 4 s group timeout, not a hang


# ------------------------------------------------------- checkpoint robustness
def test_incomplete_checkpoint_directories_are_skipped_on_resume(tmp_path):
    for n, files in ((100, 4), (200, 4), (300, 2)):  # the copy of checkpoint_300 was interrupted
        d = tmp_path / f"checkpoint_{n}"
        d.mkdir()
        for i in range(files):
            (d / f"checkpoint_{n}-model_part-0-shard{i}.pt").write_bytes(b"x")
    assert checkpoint_utils.get_latest_complete_checkpoint_dir(str(tmp_path), 4) == str(tmp_path / "checkpoint_200")
    assert checkpoint_utils.get_latest_complete_checkpoint_dir(str(tmp_path), 8) is None


def test_failed_write_leaves_no_partial_checkpoint_and_surfaces_the_error(tmp_path, monkeypatch):
    target = tmp_path / "checkpoint_5.pt"
    checkpoint_utils.write_checkpoint({"a": torch.arange(4)}, str(target), asynchronous=False)
    good = target.read_bytes()

    def broken_save(obj, f, *a, **k):
        f.write(b"partial")
        raise OSError("disk full")

    monkeypatch.setattr(torch, "save", broken_save)
    with pytest.raises(OSError):
        checkpoint_utils.write_checkpoint({"a": torch.arange(8)}, str(target), asynchronous=False)
    assert target.read_bytes() == good  # the previous complete file is untouched (write goes to .tmp, then rename)
    fut = checkpoint_utils.write_checkpoint({"a": torch.arange(8)}, str(tmp_path / "checkpoint_6.pt"), asynchronous=True)
    with pytest.raises(OSError):
        checkpoint_utils.wait_for_pending_writes()
    assert fut.done() and not (tmp_path / "checkpoint_6.pt").exists()


def test_truncated_shard_is_rejected_when_loading(tmp_path):
    path = tmp_path / "checkpoint_1.pt"
    torch.save({"model": {"w": torch.randn(64, 64)}, "cfg": None}, path)
    data = path.read_bytes()
    path.write_bytes(data[: len(data) // 2])
    with pytest.raises(Exception):
        checkpoint_utils.load_checkpoint_to_cpu(str(path))


# ------------------------------------ epoch / double-buffer protocol on CPU threads
def test_flag_in_data_exchange_never_delivers_stale_rows():
    """The exchange of ``msq_gemm_skinny_allreduce`` replayed by threads: every (rank, CTA) stores {payload, epoch}
    units into both receive buffers of every rank, alternating per product, and polls its own buffer for the
    current epoch.  Random delays let ranks run up to one product ahead of each other; a consumer must never see
    a payload of another product."""
    world, ctas, products = 3, 4, 60
    # recv[rank][parity][src][cta] = (payload, epoch); one lock-free cell per writer, like an aligned 8-byte store
    recv = [[[[(0, 0) for _ in range(ctas)] for _ in range(world)] for _ in range(2)] for _ in range(world)]
    errors = []

    def cta_thread(rank, cta, seed):
        rng = random.Random(seed)
        epoch = 0  # the per-CTA counter the kernel keeps in device memory
        for product in range(products):
            epoch += 1
            parity = product & 1
            payload = (rank, cta, product)
            for dst in range(world):
                if rng.random() < 0.3:
                    time.sleep(rng.random() * 0.002)
                recv[dst][parity][rank][cta] = (payload, epoch)
            for src in range(world):
                deadline = time.time() + 20
                while True:
                    got, e = recv[rank][parity][src][cta]
                    if e == epoch:
                        break
                    if time.time() > deadline:
                        errors.append(("timeout", rank, cta, product, src))
                        return
                    time.sleep(0)
                if got != (src, cta, product):
                    errors.append(("stale", rank, cta, product, src, got))
                    return
            if rng.random() < 0.2:
                time.sleep(rng.random() * 0.003)  # a slow consumer: peers may already be sending the next product

    threads = [threading.Thread(target=cta_thread, args=(r, c, 1000 * r + c)) for r in range(world) for c in range(ctas)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors[:3]


# --------------------------------------------------------------- rendezvous retries
def test_tcp_store_connection_is_retried_with_backoff(monkeypatch):
    """A start-up race (the store's host is not listening yet) is absorbed by retries; a persistent failure
    surfaces after the last attempt."""
    import torch.distributed as dist

    from metaseq_b200.parallel import rendezvous

    calls, sleeps = [], []

    class FlakyStore:
        def __init__(self, *a, **k):
            calls.append(a)
            if len(calls) < 3:
                raise RuntimeError("connect() timed out")

    monkeypatch.setattr(dist, "TCPStore", FlakyStore)
    monkeypatch.setattr(rendezvous.time, "sleep", sleeps.append)
    store = rendezvous._store_with_retries("127.0.0.1", 1234, 1, 2, datetime.timedelta(seconds=1))
    assert isinstance(store, FlakyStore) and len(calls) == 3
    assert len(sleeps) == 2 and sleeps[1] > sleeps[0] >= 1.0  # exponential backoff with jitter

    class DeadStore:
        def __init__(self, *a, **k):
            calls.append(a)
            raise RuntimeError("connection refused")

    calls.clear()
    monkeypatch.setattr(dist, "TCPStore", DeadStore)
    with pytest.raises(RuntimeError):
        rendezvous._store_with_retries("127.0.0.1", 1234, 1, 2, datetime.timedelta(seconds=1))
    assert len(calls) == rendezvous._MAX_RETRIES
    with pytest.raises(ValueError):
        list(rendezvous._tcpr_handler("tcpr://127.0.0.1:1234?rank=0"))  # world_size missing


def test_tcpr_rendezvous_initialises_a_process_group():
    import torch.multiprocessing as mp

    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_tcpr_rank, args=(world, _free_port(), out), nprocs=world, join=True)
        assert dict(out) == {0: 3.0, 1: 3.0}


def _tcpr_rank(rank, world, port, out):
    import torch.distributed as dist

    from metaseq_b200.parallel import rendezvous  # noqa: F401 - registers the schemes

    # torch appends rank and world_size to the URL itself
    dist.init_process_group("gloo", init_method=f"tcpr://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=30))
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t)
    out[rank] = float(t)
    dist.destroy_process_group()
