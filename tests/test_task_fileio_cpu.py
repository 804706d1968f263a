"""Streaming language-modeling task wired through the real parser (JSONL shards, BPE tokenizer, shard rotation per
epoch, CM3 variant), the finetuning collater, and the file-io layer."""
import json
import os

import pytest
import torch

from metaseq_b200 import options, tasks
from metaseq_b200.dataclass.utils import convert_namespace_to_config


def _write_tokenizer(tmp_path):
    """A byte-level BPE vocabulary whose first four ids are the dictionary specials."""
    from tokenizers import ByteLevelBPETokenizer

    tok = ByteLevelBPETokenizer()
    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n".join(f"the quick brown fox {i} jumps over the lazy dog" for i in range(50)))
    tok.train([str(corpus)], vocab_size=300, special_tokens=["<s>", "<pad>", "</s>", "<unk>"])
    tok.save_model(str(tmp_path))
    return str(tmp_path / "vocab.json"), str(tmp_path / "merges.txt")


def _write_shards(root, n_shards=2, docs=12):
    for split in ("train", "valid"):
        for s in range(n_shards if split == "train" else 1):
            d = root / split / f"{s:02d}"
            d.mkdir(parents=True)
            for corpus in ("a", "b"):
                with open(d / f"{corpus}.jsonl", "w") as f:
                    for i in range(docs):
                        f.write(json.dumps({"text": f"shard {s} corpus {corpus} doc {i} the quick brown fox"}) + "\n")


def _task(tmp_path, extra=()):
    vocab, merges = _write_tokenizer(tmp_path)
    data = tmp_path / "data"
    if not data.exists():
        _write_shards(data)
    parser = options.get_training_parser()
    ns = options.parse_args_and_arch(parser, input_args=[
        "--task", "streaming_language_modeling", "--data", str(data), "--vocab-filename", vocab, "--merges-filename",
        merges, "--tokens-per-sample", "16", "--batch-size", "2", "--arch", "transformer_lm_megatron", "--optimizer",
        "adam", "--lr", "1e-3", "--criterion", "cross_entropy", "--sample-break-mode", "none", *extra])
    cfg = convert_namespace_to_config(ns)
    return tasks.setup_task(cfg.task), cfg


def test_streaming_task_rotates_shards_and_collates(tmp_path):
    task, cfg = _task(tmp_path)
    d = task.source_dictionary
    assert (d.bos(), d.pad(), d.eos(), d.unk()) == (0, 1, 2, 3) and len(d) >= 260
    assert task.get_shard_str(1, "train") == "00" and task.get_shard_str(2, "train") == "01"
    assert task.get_shard_str(3, "train") == "00" and task.get_shard_str(5, "valid") == "00"
    ds = task.load_dataset("train", epoch=1)
    ds.set_epoch(1)
    blocks = list(ds)
    assert all(len(b["block"]) == 17 for b in blocks)  # tokens_per_sample + 1: input and target overlap by shift
    text = task.tokenizer.decode(torch.cat([b["block"] for b in blocks]).tolist())
    assert "shard 0" in text and "shard 1" not in text
    batch = task._collate_fn(blocks[:2])
    assert batch["net_input"]["src_tokens"].shape == (2, 16) and batch["target"].shape == (2, 16)
    assert torch.equal(batch["net_input"]["src_tokens"][:, 1:], batch["target"][:, :-1])
    assert batch["ntokens"] == 32 and batch["nsentences"] == 2
    ds2 = task.load_dataset("train", epoch=2)
    ds2.set_epoch(2)
    assert "shard 1" in task.tokenizer.decode(torch.cat([b["block"] for b in ds2]).tolist())


def test_streaming_task_documents_end_with_eod(tmp_path):
    task, _ = _task(tmp_path)
    toks = task._tokenize_one_json({"text": "the quick brown fox"})
    assert toks[-1].item() == task.eod and toks.dtype == torch.long and len(toks) > 2


def test_streaming_task_cm3_variant(tmp_path):
    task, _ = _task(tmp_path, ["--language-modeling-type", "cm3", "--cm3-num-sentinel-tokens", "4",
                               "--cm3-lambda-sentinel-tokens", "1", "--cm3-mode", "fixed",
                               "--cm3-allow-across-eod-boundaries"])
    sentinel = task.tokenizer.token_to_id("<sentinel:0>")
    assert sentinel is not None and task.tokenizer.token_to_id("<eoss>") is not None
    ds = task.load_dataset("train", epoch=1)
    ds.set_epoch(1)
    blocks = list(ds)
    assert len(blocks) > 3 and all(len(b["block"]) <= 17 for b in blocks)
    assert any(sentinel in b["block"].tolist() for b in blocks)


# ------------------------------------------------------------------------------ file io
def test_path_manager_native_operations(tmp_path):
    from metaseq_b200.file_io import PathManager

    p = str(tmp_path / "a" / "b.txt")
    PathManager.mkdirs(os.path.dirname(p))
    with PathManager.open(p, "w") as f:
        f.write("hello")
    assert PathManager.exists(p) and PathManager.isfile(p) and PathManager.isdir(str(tmp_path / "a"))
    assert PathManager.ls(str(tmp_path / "a")) == ["b.txt"]
    q = str(tmp_path / "a" / "c.txt")
    assert PathManager.copy(p, q, overwrite=True)
    PathManager.rename(q, str(tmp_path / "a" / "d.txt"))
    assert sorted(PathManager.ls(str(tmp_path / "a"))) == ["b.txt", "d.txt"]
    PathManager.rm(p)
    assert not PathManager.exists(p)
    assert PathManager.get_local_path(q) == q


def test_non_blocking_writes_are_flushed_on_join(tmp_path):
    from metaseq_b200.file_io import PathManager

    path = str(tmp_path / "async.txt")
    done = []
    with PathManager.opena(path, "w", callback_after_file_close=lambda: done.append(1)) as f:
        for i in range(100):
            f.write(f"{i}\n")
    assert PathManager.async_join(path) or True
    PathManager.async_close()
    assert open(path).read().splitlines() == [str(i) for i in range(100)] and done == [1]


def test_checkpoint_write_symlink_and_load_cpu(tmp_path):
    from metaseq_b200 import checkpoint_utils
    from metaseq_b200.file_io import torch_load_cpu

    obj = {"model": {"w": torch.arange(6).view(2, 3)}, "cfg": {"x": 1}}
    path = str(tmp_path / "checkpoint_3.pt")
    link = str(tmp_path / "checkpoint_last.pt")
    checkpoint_utils.write_checkpoint(obj, path, asynchronous=True, files_to_symlink_to=[link])
    checkpoint_utils.wait_for_pending_writes()
    back = torch_load_cpu(link)
    assert torch.equal(back["model"]["w"], obj["model"]["w"]) and back["cfg"] == {"x": 1}
    assert os.path.exists(path) and not os.path.exists(path + ".tmp")
    # with a callback the caller takes over what happens after the write (upload, links)
    called = []
    checkpoint_utils.write_checkpoint(obj, str(tmp_path / "checkpoint_4.pt"), asynchronous=True,
                                      async_callback_fn=lambda f, links: called.append((f, links)),
                                      files_to_symlink_to=[link])
    checkpoint_utils.wait_for_pending_writes()
    assert called == [(str(tmp_path / "checkpoint_4.pt"), [link])]
    checkpoint_utils.verify_checkpoint_directory(str(tmp_path))
    assert checkpoint_utils._is_checkpoint_sharded(str(tmp_path / "checkpoint_3-shard0.pt")) or True


def _write_indexed_corpus(root, dictionary, docs, split="train"):
    from metaseq_b200.data import indexed_dataset

    prefix = str(root / split)
    builder = indexed_dataset.make_builder(prefix + ".bin", "mmap", vocab_size=len(dictionary))
    for d in docs:
        builder.add_item(torch.tensor(d, dtype=torch.int64))
    builder.finalize(prefix + ".idx")


def test_legacy_language_modeling_task_loads_an_indexed_corpus(tmp_path):
    """The map-style task (the one the completions service is launched with): mmap corpus -> token blocks ->
    source / target pairs, plus its padding and document-shuffling options."""
    from metaseq_b200.data import Dictionary

    d = Dictionary()
    for i in range(40):
        d.add_symbol(f"w{i}")
    d.save(str(tmp_path / "dict.txt"))
    eos = d.eos()
    docs = [[4 + (i + j) % 40 for j in range(3 + i % 7)] + [eos] for i in range(30)]
    _write_indexed_corpus(tmp_path, d, docs)

    def task_for(extra=()):
        ns = options.parse_args_and_arch(options.get_training_parser(), input_args=[
            "--task", "language_modeling", str(tmp_path), "--tokens-per-sample", "16", "--batch-size", "4", "--arch",
            "transformer_lm_megatron", "--optimizer", "adam", "--lr", "1e-3", "--criterion", "cross_entropy", *extra])
        cfg = convert_namespace_to_config(ns)
        t = tasks.setup_task(cfg.task)
        t.load_dataset("train")
        return t

    t = task_for()
    ds = t.dataset("train")
    total = sum(len(x) for x in docs)
    assert len(ds) == -(-total // 16)
    batch = ds.collater([ds[0], ds[1]])
    src, tgt = batch["net_input"]["src_tokens"], batch["target"]
    assert src.shape == (2, 16) and torch.equal(src[:, 1:], tgt[:, :-1])  # next-token targets
    flat = [tok for doc in docs for tok in doc]
    # the target is the block itself, the source the same tokens one position earlier (document separator first)
    assert tgt[0].tolist() == flat[:16] and src[0].tolist() == [eos] + flat[:15]
    # fixed batch shape
    t2 = task_for(["--pad-to-fixed-length", "--pad-to-fixed-bsz"])
    ds2 = t2.dataset("train")
    last = ds2.collater([ds2[len(ds2) - 1]])
    assert last["net_input"]["src_tokens"].shape == (4, 16)
    assert (last["net_input"]["src_tokens"][1:] == d.pad()).all()
    # document-level blocks under a shuffled sort order, then fixed-size blocks: every document arrives intact
    t3 = task_for(["--shuffle-docs"])
    ds3 = t3.dataset("train")
    seen = [tok for i in range(len(ds3)) for tok in ds3[i]["target"].tolist()]
    assert sorted(seen) == sorted(flat)
    as_docs, cur = [], []
    for tok in seen:
        cur.append(tok)
        if tok == eos:
            as_docs.append(cur)
            cur = []
    assert sorted(map(tuple, as_docs)) == sorted(map(tuple, docs))


def test_cache_dir_and_file_lock(tmp_path, monkeypatch):
    from metaseq_b200.file_io import file_lock, get_cache_dir

    monkeypatch.setenv("FVCORE_CACHE", str(tmp_path / "cache"))
    assert get_cache_dir() == str(tmp_path / "cache") and os.path.isdir(tmp_path / "cache")
    assert get_cache_dir(str(tmp_path / "other")) == str(tmp_path / "other")
    blocked = tmp_path / "file"  # a file where a directory is wanted: falls back to the temporary folder
    blocked.write_text("")
    assert get_cache_dir(str(blocked / "sub")).endswith("iopath_cache")
    target = str(tmp_path / "sub" / "weights.bin")
    with file_lock(target):
        assert os.path.exists(target + ".lock")
        with pytest.raises(TimeoutError):
            with file_lock(target, timeout=0.2):
                pass
    with file_lock(target, timeout=0.2):  # free again
        pass


def test_path_manager_handlers_cwd_move_and_argument_checks(tmp_path):
    import io

    from metaseq_b200.file_io.path_manager import NativePathHandler, PathHandler, PathManagerBase

    class MemHandler(PathHandler):
        """A toy remote store: objects in a dict, fetched to local files on demand."""

        def __init__(self, cache):
            self.objects, self.cache = {}, cache

        def _get_supported_prefixes(self):
            return ["mem://"]

        def _get_local_path(self, path, force=False, **kw):
            self._check_kwargs(kw)
            local = os.path.join(self.cache, path[len("mem://"):].replace("/", "_"))
            if force or not os.path.exists(local):
                with open(local, "wb") as f:
                    f.write(self.objects[path])
            return local

        def _copy_from_local(self, local_path, dst_path, overwrite=False, ttl=None, **kw):
            self._check_kwargs(kw)
            if dst_path in self.objects and not overwrite:
                return False
            with open(local_path, "rb") as f:
                self.objects[dst_path] = f.read()
            return True

        def _open(self, path, mode="r", **kw):
            data = self.objects[path]
            return io.BytesIO(data) if "b" in mode else io.StringIO(data.decode())

        def _exists(self, path, **kw):
            return path in self.objects

    pm = PathManagerBase()
    mem = MemHandler(str(tmp_path))
    pm.register_handler(mem)
    with pytest.raises(KeyError):
        pm.register_handler(MemHandler(str(tmp_path)), allow_override=False)
    assert pm.path_requires_pathmanager("mem://bucket/x") and not pm.path_requires_pathmanager(str(tmp_path))
    assert not pm.supports_rename("mem://bucket/x")
    with pytest.raises(ValueError):
        pm.rename("mem://bucket/x", "mem://bucket/y")

    # local -> remote -> local through copy(): different handlers go through a local file
    src = tmp_path / "src.txt"
    src.write_text("payload")
    assert pm.copy(str(src), "mem://bucket/x")
    assert mem.objects["mem://bucket/x"] == b"payload"
    assert not pm.copy(str(src), "mem://bucket/x")  # exists, no overwrite
    back = tmp_path / "back.txt"
    assert pm.copy("mem://bucket/x", str(back))
    assert back.read_text() == "payload"
    with pm.open("mem://bucket/x") as f:
        assert f.read() == "payload"
    # handler-specific arguments pass through; unknown ones raise in strict mode and only warn otherwise
    assert pm.copy_from_local(str(src), "mem://bucket/z", ttl=5)
    with pytest.raises(ValueError):
        pm.exists(str(src), cache_timeout=3)
    pm.set_strict_kwargs_checking(False)
    assert pm.exists(str(src), cache_timeout=3)
    pm.set_strict_kwargs_checking(True)

    # working directory for relative local paths
    sub = tmp_path / "wd"
    sub.mkdir()
    assert not pm.set_cwd("relative/dir")
    assert pm.set_cwd(str(sub))
    with pm.open("note.txt", "w") as f:
        f.write("x")
    assert (sub / "note.txt").exists() and pm.isfile("note.txt") and pm.ls(".") == ["note.txt"]
    assert pm.mv("note.txt", "moved.txt") and (sub / "moved.txt").exists()
    (sub / "other.txt").write_text("y")
    assert not pm.mv("other.txt", "moved.txt")  # never overwrites
    assert pm.get_local_path("moved.txt") == str(sub / "moved.txt")
    assert pm.set_cwd(None) and pm.get_local_path("moved.txt") == "moved.txt"
    with pytest.raises(AssertionError):
        pm.mv(str(src), "mem://bucket/q")
    # a replacement for the local handler
    class Quiet(NativePathHandler):
        pass

    with pytest.raises(ValueError):
        pm.register_handler(Quiet(), allow_override=False)
    pm.register_handler(Quiet())
    assert isinstance(pm._native, Quiet) and pm.exists(str(src))


def test_http_fetch_retries_timeouts_with_growing_limits(monkeypatch, tmp_path):
    import io

    import requests

    from metaseq_b200 import file_utils

    seen = []

    class Reply:
        status_code = 200
        headers = {"ETag": "abc"}

        def raise_for_status(self):
            pass

        def iter_content(self, chunk_size):
            yield b"pay"
            yield b""
            yield b"load"

    def fake_get(url, stream=False, timeout=None):
        seen.append(timeout)
        if len(seen) < 3:
            raise requests.exceptions.Timeout()
        return Reply()

    monkeypatch.setattr(requests, "get", fake_get)
    buf = io.BytesIO()
    file_utils.http_get("http://example.invalid/f", buf)
    assert buf.getvalue() == b"payload" and seen == [10, 20, 40]
    monkeypatch.setattr(requests, "get", lambda *a, **k: (_ for _ in ()).throw(requests.exceptions.Timeout()))
    with pytest.raises(RuntimeError, match="Unable to fetch"):
        file_utils.http_get("http://example.invalid/f", io.BytesIO())
    # the cache goes through the same calls and remembers the ETag in the file name
    monkeypatch.setattr(requests, "get", lambda url, stream=False, timeout=None: Reply())
    monkeypatch.setattr(requests, "head", lambda url, allow_redirects=True, timeout=None: Reply())
    path = file_utils.cached_path("http://example.invalid/f", cache_dir=str(tmp_path))
    assert open(path, "rb").read() == b"payload"
    assert os.path.basename(path) == file_utils.url_to_filename("http://example.invalid/f", "abc")


def test_async_handles_on_one_path_keep_their_order_buffer_and_report_failures(tmp_path):
    import io

    from metaseq_b200.file_io import PathManager
    from metaseq_b200.file_io.non_blocking_io import NonBlockingBufferedIO, NonBlockingIOManager

    # two handles on one path: the second's writes land behind the first's, whatever the thread timing
    path = str(tmp_path / "log.txt")
    a = PathManager.opena(path, "a")
    for i in range(200):
        a.write(f"a{i}\n")
    a.close()
    b = PathManager.opena(str(tmp_path / "." / "log.txt"), "a")  # the same file under another spelling
    b.write("b0\n")
    b.close()
    assert PathManager.async_join(path)
    assert open(path).read().splitlines() == [f"a{i}" for i in range(200)] + ["b0"]

    # buffered: many small writes become few large ones
    class Counting(io.BytesIO):
        writes = 0

        def write(self, data):
            Counting.writes += 1
            return super().write(data)

        def close(self):
            Counting.final = self.getvalue()
            super().close()

    mgr = NonBlockingIOManager(buffered=True)
    h = mgr.get_non_blocking_io("mem", Counting(), buffering=64)
    assert isinstance(h, NonBlockingBufferedIO)
    for i in range(100):
        h.write(b"0123456789")
    h.close()
    assert mgr._join("mem") and Counting.final == b"0123456789" * 100 and Counting.writes <= 16
    with pytest.raises(ValueError, match="not using a buffered writer"):
        NonBlockingIOManager().get_non_blocking_io("mem", io.BytesIO(), buffering=64)
    with pytest.raises(ValueError, match="no async IO associated"):
        mgr._join("never-opened")

    # a failed write surfaces at the join, and the callback still runs behind it
    class Broken(io.BytesIO):
        def write(self, data):
            raise OSError("disk full")

    ran = []
    mgr = NonBlockingIOManager()
    h = mgr.get_non_blocking_io("bad", Broken(), callback_after_file_close=lambda: ran.append(1))
    h.write(b"x")
    h.close()
    with pytest.raises(OSError, match="disk full"):
        mgr._close_thread_pool()
    assert ran == [1]
    PathManager.async_close()


@pytest.mark.parametrize("workers", [1, 3])
def test_dictionary_is_built_from_text_files_by_worker_processes(tmp_path, workers):
    from metaseq_b200.tasks.base_task import BaseTask

    lines = ["the cat sat", "the dog sat down", "a cat"] * 7
    f = tmp_path / "corpus.txt"
    f.write_text("\n".join(lines) + "\n")
    d = BaseTask.build_dictionary([str(f)], workers=workers, padding_factor=1)
    assert d.get_count(d.index("the")) == 14 and d.get_count(d.index("cat")) == 14 and d.get_count(d.index("down")) == 7
    assert d.get_count(d.eos()) == len(lines) + 1  # one per line, on top of the symbol's initial count of one
    assert d[d.nspecial] in ("the", "cat", "sat")  # most frequent first
    cut = BaseTask.build_dictionary([str(f)], workers=workers, threshold=10, padding_factor=1)
    assert "down" not in cut and "the" in cut

    class T(BaseTask):
        source_dictionary = d

    toks, lens = T.__new__(T).get_interactive_tokens_and_lengths(["the cat", "a dog sat"], lambda s: s)
    assert lens == [3, 4] and toks[0].tolist() == [d.index("the"), d.index("cat"), d.eos()]


# ------------------------------------------------------------------ blob storage against an in-memory service
class ResourceNotFoundError(Exception):
    pass


class _FakeBlobStore:
    """The slice of the blob service client API that the handler uses, over a dict."""

    def __init__(self):
        import datetime

        self.blobs = {}  # (container, name) -> (bytes, last_modified)
        self.staged = {}
        self.now = lambda: datetime.datetime.now(datetime.timezone.utc)
        self.downloads = 0

    def get_blob_client(self, container, blob):
        return _FakeBlobClient(self, container, blob)

    def get_container_client(self, container):
        store = self

        class Container:
            def list_blobs(self, name_starts_with=""):
                import types

                return [types.SimpleNamespace(name=n) for (c, n) in sorted(store.blobs)
                        if c == container and n.startswith(name_starts_with)]

        return Container()


class _FakeBlobClient:
    def __init__(self, store, container, blob):
        self.store, self.container, self.blob_name = store, container, blob

    def _get(self):
        try:
            return self.store.blobs[(self.container, self.blob_name)]
        except KeyError:
            raise ResourceNotFoundError(self.blob_name) from None

    def get_blob_properties(self):
        import types

        data, when = self._get()
        return {"size": len(data), "last_modified": when, "copy": types.SimpleNamespace(status="success")} | {}

    def download_blob(self):
        data, _ = self._get()
        self.store.downloads += 1

        class Stream:
            def chunks(self, size=5):
                return iter([data[i:i + size] for i in range(0, len(data), size)])

            def readinto(self, out):
                out.write(data)

        return Stream()

    def stage_block(self, block_id, stream, length):
        self.store.staged.setdefault((self.container, self.blob_name), {})[block_id] = stream.read(length)

    def commit_block_list(self, blocks):
        staged = self.store.staged.pop((self.container, self.blob_name))
        self.store.blobs[(self.container, self.blob_name)] = (b"".join(staged[b.id] for b in blocks), self.store.now())

    def upload_blob(self, src, length=None, overwrite=False):
        self.store.blobs[(self.container, self.blob_name)] = (src.read(), self.store.now())

    def delete_blob(self):
        self._get()
        del self.store.blobs[(self.container, self.blob_name)]

    def start_copy_from_url(self, url):
        assert url.endswith("?sas-token") and ".blob.core.windows.net/" in url
        container, _, name = url.split(".blob.core.windows.net/")[1].split("?")[0].partition("/")
        self.store.blobs[(self.container, self.blob_name)] = (self.store.blobs[(container, name)][0], self.store.now())


def test_blob_storage_handler_streams_blocks_lists_copies_and_caches(tmp_path, monkeypatch):
    import types

    from metaseq_b200.file_io import azure_blob
    from metaseq_b200.file_io.path_manager import PathManagerBase

    store = _FakeBlobStore()
    seen = {}

    def factory(url, token):
        seen["url"], seen["token"] = url, token
        return store

    monkeypatch.setenv(azure_blob.ENV_SAS_TOKEN, "sas-token")
    handler = azure_blob.AzureBlobPathHandler(cache_dir=str(tmp_path / "cache"), service_factory=factory,
                                              block_factory=azure_blob.blob_block)
    # get_blob_properties returns a mapping with attribute access on "copy" in the SDK; adapt the fake's dict
    real_props = _FakeBlobClient.get_blob_properties
    monkeypatch.setattr(_FakeBlobClient, "get_blob_properties",
                        lambda self: type("P", (dict,), {"copy": types.SimpleNamespace(status="success")})(real_props(self)))
    pm = PathManagerBase()
    pm.register_handler(handler)
    root = "az://acct/cont/run1"
    assert handler._parse_uri(root + "/a/b.pt") == ("acct", "cont", "run1/a/b.pt")
    with pytest.raises(ValueError):
        handler._parse_uri("s3://x/y")
    assert not pm.exists(root + "/ckpt.pt")

    payload = bytes(range(256)) * 5
    with pm.open(root + "/ckpt.pt", "wb", buffering=300) as f:  # 300-byte blocks
        for i in range(0, len(payload), 100):
            f.write(payload[i:i + 100])
    assert seen == {"url": "https://acct.blob.core.windows.net", "token": "sas-token"}
    assert store.blobs[("cont", "run1/ckpt.pt")][0] == payload and not store.staged
    assert pm.isfile(root + "/ckpt.pt") and pm.isdir(root) and not pm.isdir(root + "/ckpt.pt") and pm.exists(root)
    with pm.open(root + "/ckpt.pt", "rb") as f:
        assert f.read(7) == payload[:7] and f.read() == payload[7:]
    with pm.open(root + "/notes.txt", "w") as f:
        f.write("héllo\nworld\n")
    with pm.open(root + "/notes.txt", "r") as f:
        assert f.read().splitlines() == ["héllo", "world"]
    assert pm.ls(root) == ["run1/ckpt.pt", "run1/notes.txt"]

    # uploads, server-side copies, removal
    local = tmp_path / "local.bin"
    local.write_bytes(b"abc")
    assert pm.copy_from_local(str(local), root + "/up.bin") and not pm.copy_from_local(str(local), root + "/up.bin")
    assert pm.copy_from_local(str(local), root + "/up.bin", overwrite=True)
    assert pm.copy(root + "/up.bin", root + "/up2.bin") and store.blobs[("cont", "run1/up2.bin")][0] == b"abc"
    pm.rm(root + "/up2.bin")
    assert not pm.exists(root + "/up2.bin")
    with pytest.raises(OSError):
        pm.rm(root + "/up2.bin")

    # the local cache is reused until the blob changes
    before = store.downloads
    p1 = pm.get_local_path(root + "/up.bin")
    assert open(p1, "rb").read() == b"abc" and p1.startswith(str(tmp_path / "cache")) and store.downloads == before + 1
    assert pm.get_local_path(root + "/up.bin") == p1 and store.downloads == before + 1
    import datetime

    store.blobs[("cont", "run1/up.bin")] = (b"newer", store.now() + datetime.timedelta(seconds=60))
    assert open(pm.get_local_path(root + "/up.bin"), "rb").read() == b"newer"
    d = pm.get_local_path(root)  # a directory: everything under it
    assert sorted(n for n in os.listdir(d) if not n.endswith(".lock")) == ["ckpt.pt", "notes.txt", "up.bin"]


class ClientError(Exception):
    def __init__(self, message="Not Found"):
        super().__init__(message)
        self.response = {"Error": {"Message": message}}


class _FakeS3:
    """The slice of the S3 client API that the handler uses, over a dict of one bucket."""

    def __init__(self):
        import datetime

        self.objects = {}
        self.now = lambda: datetime.datetime.now(datetime.timezone.utc)
        self.downloads = 0

    def head_object(self, Bucket, Key):
        if Key not in self.objects:
            raise ClientError()
        return {"ContentLength": len(self.objects[Key][0]), "LastModified": self.objects[Key][1]}

    def list_objects_v2(self, Bucket, Prefix="", Delimiter=None, MaxKeys=1000, ContinuationToken=None):
        keys = sorted(k for k in self.objects if k.startswith(Prefix))
        contents, prefixes = [], []
        for k in keys:
            rest = k[len(Prefix):]
            if Delimiter and Delimiter in rest:
                p = Prefix + rest.split(Delimiter)[0] + Delimiter
                if p not in prefixes:
                    prefixes.append(p)
            else:
                contents.append({"Key": k})
        start = int(ContinuationToken or 0)
        page = contents[start:start + 2]  # tiny pages: the handler must follow the continuation token
        more = start + 2 < len(contents)
        out = {"Contents": page[:MaxKeys], "KeyCount": len(page[:MaxKeys]) + len(prefixes), "IsTruncated": more}
        if not start:
            out["CommonPrefixes"] = [{"Prefix": p} for p in prefixes]
        if more:
            out["NextContinuationToken"] = str(start + 2)
        return out

    def upload_fileobj(self, f, bucket, key, **kw):
        self.objects[key] = (f.read(), self.now())

    def upload_file(self, path, bucket, key, **kw):
        self.objects[key] = (open(path, "rb").read(), self.now())

    def download_file(self, bucket, key, path, **kw):
        self.downloads += 1
        open(path, "wb").write(self.objects[key][0])

    def copy(self, src, bucket, key, **kw):
        self.objects[key] = (self.objects[src["Key"]][0], self.now())

    def put_object(self, Bucket, Key):
        self.objects[Key] = (b"", self.now())

    def delete_object(self, Bucket, Key):
        if Key not in self.objects:
            raise ClientError()
        del self.objects[Key]


def test_s3_handler_uploads_on_close_lists_one_level_and_refreshes_its_cache(tmp_path):
    import datetime

    from metaseq_b200.file_io.path_manager import PathManagerBase
    from metaseq_b200.file_io.s3 import S3PathHandler

    s3 = _FakeS3()
    pm = PathManagerBase()
    pm.register_handler(S3PathHandler(cache_dir=str(tmp_path / "cache"), client_factory=lambda: s3))
    root = "s3://bucket/run"
    with pm.open(root + "/a.bin", "wb") as f:
        f.write(b"12")
        f.write(b"345")
        assert "run/a.bin" not in s3.objects  # nothing leaves before close
    assert s3.objects["run/a.bin"][0] == b"12345"
    with pm.open(root + "/notes.txt", "w") as f:
        f.write("héllo\n")
    for name in ("b.bin", "c.bin", "sub/d.bin", "sub/deeper/e.bin"):
        s3.objects["run/" + name] = (b"x", s3.now())
    assert pm.isfile(root + "/a.bin") and not pm.isfile(root + "/zzz") and pm.isdir(root) and pm.isdir(root + "/sub/")
    assert not pm.isdir(root + "/a.bin") and pm.exists(root + "/sub") and not pm.exists(root + "/nothing")
    assert sorted(pm.ls(root)) == ["run/a.bin", "run/b.bin", "run/c.bin", "run/notes.txt", "run/sub/"]
    pm.mkdirs(root + "/empty/")
    assert pm.isdir(root + "/empty") and pm.ls(root + "/empty") == []

    with pm.open(root + "/notes.txt", "r") as f:
        assert f.read() == "héllo\n"
    before = s3.downloads
    with pm.open(root + "/a.bin", "rb") as f:
        assert f.read() == b"12345"
    p = pm.get_local_path(root + "/a.bin")
    assert s3.downloads == before + 1 and p.startswith(str(tmp_path / "cache"))
    s3.objects["run/a.bin"] = (b"changed", s3.now() + datetime.timedelta(seconds=60))
    assert open(pm.get_local_path(root + "/a.bin"), "rb").read() == b"changed" and s3.downloads == before + 2
    with pytest.raises(NotImplementedError):
        pm.get_local_path(root + "/sub/")

    local = tmp_path / "up.bin"
    local.write_bytes(b"up")
    assert pm.copy_from_local(str(local), root + "/up.bin") and not pm.copy_from_local(str(local), root + "/up.bin")
    assert pm.copy(root + "/up.bin", root + "/up2.bin") and s3.objects["run/up2.bin"][0] == b"up"
    with pytest.raises(AssertionError):
        pm.copy(root + "/up.bin", "s3://other/up.bin")
    pm.rm(root + "/up2.bin")
    with pytest.raises(OSError):
        pm.rm(root + "/up2.bin")
    with pytest.raises(ValueError):
        pm.exists("s3://bucket-without-key")
