"""Small modules kept for API parity with the reference: each is exercised once so that a broken import or
signature shows up here and not at a user."""
import os
import pickle

import numpy as np
import torch


def test_file_chunker_splits_a_file_on_line_boundaries(tmp_path):
    from metaseq_b200.file_chunker_utils import Chunker, find_offsets

    path = tmp_path / "corpus.txt"
    lines = [f"line {i} " + "x" * (i % 17) for i in range(200)]
    path.write_text("\n".join(lines) + "\n")
    offsets = find_offsets(str(path), 4)
    assert len(offsets) == 5 and offsets[0] == 0 and offsets[-1] == os.path.getsize(path)
    seen = []
    for a, b in zip(offsets[:-1], offsets[1:]):
        with Chunker(str(path), a, b) as it:
            seen += [ln.rstrip("\n") for ln in it]
    assert seen == lines


def test_file_utils_resolves_local_paths_and_names_cache_entries(tmp_path):
    from metaseq_b200 import file_utils

    p = tmp_path / "model.bin"
    p.write_bytes(b"x")
    assert file_utils.cached_path(str(p)) == str(p)
    assert file_utils.split_s3_path("s3://bucket/some/key.pt") == ("bucket", "some/key.pt")
    a, b = file_utils.url_to_filename("https://h/x.bin"), file_utils.url_to_filename("https://h/x.bin", etag="v2")
    assert a != b and b.startswith(a)


def test_incremental_state_mixin_keeps_per_module_entries_apart():
    from metaseq_b200.incremental_decoding_utils import with_incremental_state

    @with_incremental_state
    class Cell(torch.nn.Module):
        pass

    a, b = Cell(), Cell()
    state = {}
    a.set_incremental_state(state, "k", {"v": torch.ones(1)})
    b.set_incremental_state(state, "k", {"v": torch.zeros(1)})
    assert float(a.get_incremental_state(state, "k")["v"]) == 1.0 and float(b.get_incremental_state(state, "k")["v"]) == 0.0
    assert a.get_incremental_state(None, "k") is None and len(state) == 2


def test_feedforward_module_matches_its_function_form():
    from metaseq_b200.modules.feedforward import FeedForward, FeedForwardFn

    torch.manual_seed(0)
    fc1, fc2 = torch.nn.Linear(8, 16), torch.nn.Linear(16, 8)
    x = torch.randn(3, 8)
    ff = FeedForward(fc1, torch.relu, fc2, model_parallel=False)
    want = fc2(torch.relu(fc1(x)))
    assert torch.allclose(ff(x), want)
    # the function form takes tensor-parallel linears, which return (output, bias)
    got = FeedForwardFn(x, lambda t: (fc1(t), None), torch.relu, lambda t: (fc2(t), None))
    got = got[0] if isinstance(got, tuple) else got
    assert torch.allclose(got, want)


def test_fused_adam_names_resolve_to_the_adam_update():
    from metaseq_b200.optim.adam import Adam
    from metaseq_b200.optim.fused_adam import FusedAdamV1, get_fused_adam_class

    assert get_fused_adam_class() is not None
    torch.manual_seed(0)
    w1 = torch.nn.Parameter(torch.randn(5))
    w2 = torch.nn.Parameter(w1.detach().clone())
    a, b = FusedAdamV1([w1], lr=0.1, betas=(0.9, 0.95), weight_decay=0.1), Adam([w2], lr=0.1, betas=(0.9, 0.95), weight_decay=0.1)
    for _ in range(3):
        for w, o in ((w1, a), (w2, b)):
            w.grad = w.detach() * 0.5 + 1
            o.step()
    assert torch.allclose(w1, w2, atol=1e-6)


def test_global_memory_buffer_reuses_storage():
    from metaseq_b200.parallel.global_vars import get_global_memory_buffer

    buf = get_global_memory_buffer()
    a = buf.get_tensor((4, 8), torch.float32, "mpu", device="cpu")
    b = buf.get_tensor((2, 8), torch.float32, "mpu", device="cpu")
    assert a.shape == (4, 8) and b.shape == (2, 8) and a.data_ptr() == b.data_ptr()
    c = buf.get_tensor((16, 8), torch.float32, "mpu", device="cpu")
    assert c.shape == (16, 8)


def test_plasma_array_and_view_survive_pickling(tmp_path):
    from metaseq_b200.data.plasma_utils import PlasmaArray, PlasmaView

    big = np.arange(200_000, dtype=np.int64)
    arr = PlasmaArray(big)
    clone = pickle.loads(pickle.dumps(arr))
    assert np.array_equal(clone.array, big)
    view = PlasmaView(big, "train", (1, 2, 3), plasma_path=str(tmp_path / "plasma"))
    again = pickle.loads(pickle.dumps(view))
    assert len(again) == len(big) and np.array_equal(again.array[:10], big[:10])
    assert PlasmaView.get_object_id("train", (1, 2, 3)) == PlasmaView.get_object_id("train", (1, 2, 3))
    assert PlasmaView.get_object_id("train", (1, 2, 3)) != PlasmaView.get_object_id("valid", (1, 2, 3))


def test_single_purpose_dataset_wrappers():
    from metaseq_b200.data import append_token_dataset, id_dataset, list_dataset, numel_dataset, pad_dataset, \
        prepend_token_dataset, sort_dataset, strip_token_dataset

    base = list_dataset.ListDataset([torch.tensor([5, 6, 7]), torch.tensor([8, 9])], sizes=[3, 2])
    pre = prepend_token_dataset.PrependTokenDataset(base, token=0)
    app = append_token_dataset.AppendTokenDataset(pre, token=2)
    assert app[1].tolist() == [0, 8, 9, 2] and list(app.sizes) == [5, 4]
    stripped = strip_token_dataset.StripTokenDataset(app, id_to_strip=2)
    assert stripped[0].tolist() == [0, 5, 6, 7]
    assert numel_dataset.NumelDataset(app)[0] == 5
    assert id_dataset.IdDataset()[3] == 3
    padded = pad_dataset.RightPadDataset(app, pad_idx=1).collater([app[0], app[1]])
    assert padded.tolist() == [[0, 5, 6, 7, 2], [0, 8, 9, 2, 1]]
    order = sort_dataset.SortDataset(app, sort_order=[[1, 0]]).ordered_indices()
    assert list(order) == [1, 0]
