"""Small modules kept for API parity with the reference: each is exercised once so that a broken import or
signature shows up here and not at a user."""
import os
import pickle

import numpy as np
import pytest
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
    # multi-byte text: a seek may land inside a character, the chunks still meet on line starts
    wide = tmp_path / "wide.txt"
    rows = ["naïve café ✓ " * (1 + i % 5) + str(i) for i in range(120)]
    wide.write_text("\n".join(rows) + "\n", encoding="utf-8")
    cuts = find_offsets(str(wide), 7)
    got = []
    for a, b in zip(cuts[:-1], cuts[1:]):
        with Chunker(str(wide), a, b) as it:
            got += [ln.rstrip("\n") for ln in it]
    assert got == rows


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


def test_faster_transformer_driver_passes_sampling_parameters_and_strips_special_tokens(tmp_path):
    """The prompt loop for an external FasterTransformer build, run against a stand-in for the library's op."""
    from metaseq_b200.cli import interactive_ft as ift

    calls = {}

    class FakeOp:
        def __init__(self, *ctor):
            calls["ctor"] = ctor

        def forward(self, batch, lengths, output_length, beam_width, *rest):
            calls["forward"] = (batch.clone(), lengths.clone(), output_length, beam_width, rest)
            rows = []
            for row, n in zip(batch, lengths):
                # prompt, three new tokens, EOS, then garbage that must not be returned
                rows.append(torch.cat([row[: int(n)], torch.tensor([40, 41, 42, ift.EOS, 77, 78], dtype=torch.int32)]))
            width = max(len(r) for r in rows)
            out = torch.full((len(rows), beam_width, width), ift.PAD, dtype=torch.int32)
            for i, r in enumerate(rows):
                out[i, 0, : len(r)] = r
            return out, torch.tensor([[len(r)] * beam_width for r in rows], dtype=torch.int32)

    class FakeLib:
        ParallelGptOp = FakeOp

    weights = tmp_path / "part-0.pt"
    torch.save({"weights": [torch.ones(2, 2), torch.zeros(3)], "int8_weights": [torch.ones(2, dtype=torch.int8)],
                "int8_scales": [torch.ones(1)]}, weights)
    model = ift.build_model(FakeLib, str(weights), num_layers=2, num_heads=4, embed_size=32, vocab_size=100,
                            tensor_para_size=1, dtype=torch.bfloat16, int8_mode=1, device="cpu")
    ctor = calls["ctor"]
    assert ctor[:4] == (4, 8, 128, 2) and ctor[5] == 100 and ctor[10] == 1
    assert ctor[16][0].dtype == torch.bfloat16 and len(ctor[17]) == 1 and len(ctor[18]) == 1
    # int8 mode without int8 tensors in the file falls back to 0
    torch.save([torch.ones(2, 2)], weights)
    ift.build_model(FakeLib, str(weights), 2, 4, 32, 100, 1, int8_mode=1, device="cpu")
    assert calls["ctor"][10] == 0 and calls["ctor"][17] == []

    args = ift.get_parser().parse_args(["--weight-path", "x", "--beam-width", "2", "--top-k", "7", "--len-penalty", "0.3",
                                        "--diversity-rate", "0.1", "--repetition-penalty", "1.5", "--output-length", "4"])
    out = ift.generate(model, [[10, 11, 12], [20]], device="cpu", **ift.sampling_kwargs(args))
    assert out == [[10, 11, 12, 40, 41, 42], [20, 40, 41, 42]]  # prompt and continuation, nothing past the EOS
    batch, lengths, output_length, beam_width, rest = calls["forward"]
    assert batch[:, 0].tolist() == [ift.EOS, ift.EOS] and lengths.tolist() == [4, 2] and batch[1, 2:].tolist() == [ift.PAD] * 2
    assert output_length == 4 and beam_width == 2
    top_k, top_p, diversity, temperature, len_penalty, repetition, presence, min_length, seed, bad_words, cum = rest
    assert int(top_k) == 7 and top_k.dtype == torch.int32 and float(top_p) == pytest.approx(0.95)
    assert float(diversity) == pytest.approx(0.1) and float(len_penalty) == pytest.approx(0.3)
    assert float(repetition) == pytest.approx(1.5) and float(temperature) == pytest.approx(0.7)
    assert presence is None and min_length is None and int(seed) == 0 and bad_words is None and cum == 0


def test_reference_utility_helpers():
    from metaseq_b200 import checkpoint_utils, hub_utils, utils
    from metaseq_b200.data import data_utils

    assert utils.split_paths("/a:/b") == ["/a", "/b"] and utils.split_paths("s3://x|s3://y") == ["s3://x", "s3://y"]
    assert utils.get_perplexity(3.0) == 8.0 and utils.get_perplexity(None) == 0.0 and utils.get_perplexity(1e9) == float("inf")
    assert utils.get_precise_epoch(2, 4, 10) == pytest.approx(1.5) and utils.get_precise_epoch(None, 4, 10) is None
    assert utils.get_model_init_dtype(type("A", (), {"memory_efficient_fp16": True, "bf16": True})) == torch.bfloat16
    assert utils.get_model_init_dtype(type("A", (), {"inference": True})) == torch.float16
    assert utils.get_model_init_dtype(type("A", (), {})) == torch.float32
    t = utils.fill_with_neg_inf(torch.zeros(3, dtype=torch.float16))
    assert t.dtype == torch.float16 and torch.isinf(t).all()
    # limits: numbers, tuples, dicts, None
    assert utils.resolve_max_positions(1024, (2048, 512), None) == (1024, 512)
    assert utils.resolve_max_positions({"a": 5, "b": None}, {"a": 7, "b": 3, "c": 1}) == {"a": 5, "b": 3, "c": 1}
    assert utils.resolve_max_positions(None, None) is None
    # seeding by rank and update: reproducible inside, outer stream untouched
    torch.manual_seed(0)
    before = torch.get_rng_state()
    with utils.set_rank_seed(3, 2) as seed:
        a, n = torch.rand(2), np.random.rand()
    with utils.set_rank_seed(3, 2):
        b, m = torch.rand(2), np.random.rand()
    assert seed == 5 and torch.equal(a, b) and n == m and torch.equal(before, torch.get_rng_state())
    state = utils.get_rng_state()
    x = torch.rand(1)
    utils.set_rng_state(state)
    assert torch.equal(x, torch.rand(1))
    assert float(utils.multi_tensor_l2_total_norm([torch.ones(4), torch.ones(5)])) == pytest.approx(3.0)
    # alignments
    attn = torch.tensor([[0.1, 0.8, 0.1], [0.6, 0.3, 0.1], [0.3, 0.3, 0.4]])
    src, tgt = torch.tensor([5, 6, 2]), torch.tensor([7, 8, 2])
    assert utils.extract_hard_alignment(attn, src, tgt, pad=1, eos=2) == [(1, 0), (0, 1)]
    soft = utils.extract_soft_alignment(attn, src, tgt, pad=1, eos=2)
    assert len(soft) == 3 and soft[0] == ["0.100000", "0.800000", "0.100000"]
    assert utils.get_token_to_word_mapping([5, 2, 6], [2]) == {0: 1, 1: 1, 2: 2}
    # data helpers
    rejected = []
    assert list(data_utils.collect_filtered(lambda v: v % 2 == 0, range(5), rejected)) == [0, 2, 4] and rejected == [1, 3]
    assert data_utils.post_process("\u2581he llo \u2581wor ld", "sentencepiece") == "hello world"
    assert data_utils.post_process("a b", "none") == "a b" and data_utils.post_process("a b", None) == "a b"
    with pytest.raises(NotImplementedError):
        data_utils.post_process("a", "bogus")
    assert checkpoint_utils.is_singleton_tensor(torch.tensor(1.0)) and not checkpoint_utils.is_singleton_tensor(torch.ones(1))

    class Tok:
        def encode(self, prompt):
            return type("E", (), {"ids": [5, 6]})

        def decode(self, ids):
            return "\u0120there" if ids == [2] else "?"

    assert hub_utils.tensorize_input(Tok(), "x").tolist() == [[0, 5, 6]]
    assert hub_utils.get_next_token(torch.tensor([[[0.0, 0.0, 1.0]]]), Tok()) == "there"


def test_unlisted_numbered_validation_sets_are_an_error_unless_combined_or_ignored(tmp_path):
    from metaseq_b200.data import data_utils
    from metaseq_b200.dataclass.utils import Cfg

    for name in ("train.bin", "valid.bin", "valid.idx", "valid1.bin", "valid1.idx", "valid2.bin"):
        (tmp_path / name).write_bytes(b"")

    def cfg(**ds):
        base = {"ignore_unused_valid_subsets": False, "combine_valid_subsets": None, "disable_validation": False,
                "valid_subset": "valid"}
        base.update(ds)
        return Cfg({"dataset": Cfg(base), "task": Cfg({"data": str(tmp_path)})})

    with pytest.raises(ValueError, match=r"valid1.*valid2"):
        data_utils.raise_if_valid_subsets_unintentionally_ignored(cfg())
    data_utils.raise_if_valid_subsets_unintentionally_ignored(cfg(valid_subset="valid,valid1,valid2"))
    data_utils.raise_if_valid_subsets_unintentionally_ignored(cfg(ignore_unused_valid_subsets=True))
    data_utils.raise_if_valid_subsets_unintentionally_ignored(cfg(combine_valid_subsets=True))
    data_utils.raise_if_valid_subsets_unintentionally_ignored(cfg(disable_validation=True))


def test_old_checkpoints_are_pruned_by_public_helper(tmp_path):
    from metaseq_b200 import checkpoint_utils
    from metaseq_b200.dataclass.utils import Cfg

    for n in (10, 20, 30):
        (tmp_path / f"checkpoint_{n}-model_part-0.pt").write_bytes(b"")
        (tmp_path / f"checkpoint_{n}-model_part-1.pt").write_bytes(b"")
    cfg = Cfg({"save_dir": str(tmp_path), "keep_last_updates": 2, "keep_last_epochs": -1})
    checkpoint_utils.delete_old_checkpoint_files(cfg, end_of_epoch=False, suffix="-model_part-0")
    assert sorted(os.listdir(tmp_path)) == ["checkpoint_10-model_part-1.pt", "checkpoint_20-model_part-0.pt",
                                            "checkpoint_20-model_part-1.pt", "checkpoint_30-model_part-0.pt",
                                            "checkpoint_30-model_part-1.pt"]


def test_truncated_dictionary_multiple_pad_dataset_and_model_name():
    import metaseq_b200.models as models
    from metaseq_b200.data import Dictionary, TruncatedDictionary
    from metaseq_b200.data.pad_dataset import MultiplePadDataset

    d = Dictionary()
    for w in "abcdef":
        d.add_symbol(w)
    t = TruncatedDictionary(d, 6)
    assert len(t) == 6 and len(d) == 10 and isinstance(t, Dictionary)
    assert t[5] == d[5] and t[7] == d.unk() and t.index("a") == d.index("a") and t.pad() == d.pad()

    class Items(torch.utils.data.Dataset):
        def __init__(self, items):
            self.items, self.sizes = items, np.array([len(i) for i in items])

        def __getitem__(self, i):
            return self.items[i]

        def __len__(self):
            return len(self.items)

    ds = MultiplePadDataset(Items([torch.arange(5), torch.arange(8), torch.arange(9)]), pad_idx=1, multiple=8)
    assert ds[0].tolist() == [0, 1, 2, 3, 4, 1, 1, 1] and ds[1].numel() == 8 and ds[2].numel() == 16
    batch = ds.collater([torch.arange(5), torch.arange(9)])
    assert batch.shape == (2, 16) and batch[0, 5:].eq(1).all() and batch[1, 9:].eq(1).all()
    assert "transformer_lm" in models.MODEL_REGISTRY and "model_parallel_transformer_lm" in models.MODEL_REGISTRY


def test_weight_statistics_are_logged_at_debug_level(caplog):
    import logging

    from metaseq_b200.models.transformer_decoder import log_weight_stats

    with caplog.at_level(logging.DEBUG, logger="metaseq_b200.models.transformer_decoder"):
        log_weight_stats(torch.tensor([1.0, 3.0]), "probe")
    assert "probe, mean: 2.00000" in caplog.text and "max: 3.00000" in caplog.text


def test_plain_python_byte_level_bpe_agrees_with_the_tokenizers_library(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    from metaseq_b200.data.encoders.gpt2_bpe_utils import bytes_to_unicode, get_encoder, get_pairs

    table = bytes_to_unicode()
    assert len(table) == 256 and len(set(table.values())) == 256 and table[ord("A")] == "A" and table[32] == "Ġ"
    assert get_pairs(("a", "b", "c", "b", "c")) == {("a", "b"), ("b", "c"), ("c", "b")}

    corpus = tmp_path / "corpus.txt"
    corpus.write_text("the quick brown fox jumps over the lazy dog\nthe dog's bark: 123 4567!  we'll see naïve café\n" * 20,
                      encoding="utf-8")
    tok = tokenizers.ByteLevelBPETokenizer()
    tok.train([str(corpus)], vocab_size=400, min_frequency=1, show_progress=False)
    tok.save_model(str(tmp_path))
    enc = get_encoder(str(tmp_path / "vocab.json"), str(tmp_path / "merges.txt"))
    for text in ["the quick brown fox", "we'll see 4567 dogs!", "  two  spaces\nand a newline", "naïve café — ünïcödé ✓",
                 "unseen wordzzz"]:
        ids = enc.encode(text)
        assert ids == tok.encode(text).ids, text
        assert enc.decode(ids) == text
    assert len(enc.cache) > 0


def test_adaptive_softmax_tied_to_adaptive_input_bands():
    from metaseq_b200.modules.adaptive_softmax import AdaptiveSoftmax, TiedHeadModule

    torch.manual_seed(0)
    V, D, cutoff = 30, 16, [10, 20]

    class Bands:
        """Embedding and projection weights of three bands, as an adaptive input layer would expose them."""

        def __init__(self):
            dims = [16, 4, 1]
            sizes = [10, 10, 10]
            self.emb = [torch.nn.Parameter(torch.randn(n, d)) for n, d in zip(sizes, dims)]
            self.proj = [torch.nn.Parameter(torch.randn(D, d)) for d in dims]

        def weights_for_band(self, band):
            return self.emb[band], self.proj[band]

    bands = Bands()
    asm = AdaptiveSoftmax(V, D, cutoff, dropout=0.0, adaptive_inputs=bands, tie_proj=True)
    assert isinstance(asm.head, TiedHeadModule) and asm.head.out_dim == 10 + 2
    before = [w.clone() for w in bands.emb + bands.proj]
    x = torch.randn(2, 3, D)
    lp = asm.get_log_prob(x, None)
    assert lp.shape == (2, 3, V) and torch.allclose(lp.exp().sum(-1), torch.ones(2, 3), atol=1e-5)
    # word logits of the head are the first band's embeddings applied to the input; the tied tensors were not re-initialised
    head = asm.head(x)
    assert torch.allclose(head[:, :10], x.reshape(-1, D) @ bands.emb[0].t(), atol=1e-5)
    assert all(torch.equal(a, b) for a, b in zip(before, bands.emb + bands.proj))
    # the first tail: input -> projection transposed (tied) -> band-1 embeddings
    tail = asm.tail[0](x.reshape(-1, D))
    assert torch.allclose(tail, (x.reshape(-1, D) @ bands.proj[1]) @ bands.emb[1].t(), atol=1e-4)
    # the loss path sees the same parameters
    target = torch.tensor([[1, 12, 25], [3, 29, 11]])
    logits, targets = asm(x, target)
    loss = sum(torch.nn.functional.cross_entropy(lg, tg) for lg, tg in zip(logits, targets) if lg is not None)
    loss.backward()
    assert bands.emb[0].grad is not None and bands.emb[2].grad is not None and bands.proj[1].grad is not None


def test_config_helper_names_of_the_reference():
    from metaseq_b200.dataclass.constants import AttentionVariants, ChoiceEnum
    from metaseq_b200.dataclass.utils import (Cfg, convert_namespace_to_config, convert_namespace_to_omegaconf,
                                              merge_with_parent, overwrite_keys_not_present)
    from metaseq_b200.optim.adam import MetaseqAdamConfig

    assert convert_namespace_to_omegaconf is convert_namespace_to_config
    merged = merge_with_parent(MetaseqAdamConfig(), Cfg({"adam_eps": 1e-6, "legacy_key": 3}))
    assert merged.adam_eps == 1e-6 and merged.weight_decay == 0.0 and merged.legacy_key == 3
    cfg = Cfg({"model": Cfg({"a": 1})})
    overwrite_keys_not_present(cfg, {"model": {"a": 9, "b": 2}, "absent": {"x": 1}})
    assert dict(cfg.model) == {"a": 1, "b": 2} and "absent" not in cfg
    Choice = ChoiceEnum(["json", "none"])
    assert Choice.json == "json" and str(Choice.none) == "none" and {Choice.json: 1}[Choice.json] == 1
    assert [v.value for v in AttentionVariants] == ["default", "xformers_default"]


def test_tensor_parallel_parts_are_recut_in_memory():
    from metaseq_b200.checkpoint.reshard_mp import find_num_parts, get_n_layers, reshard_megatron_parts

    torch.manual_seed(0)
    D, F, V = 8, 16, 12
    whole = {"decoder.embed_tokens.weight": torch.randn(V, D), "decoder.embed_positions.weight": torch.randn(6, D),
             "decoder.layers.0.self_attn.qkv_proj.weight": torch.randn(3 * D, D),
             "decoder.layers.0.self_attn.qkv_proj.bias": torch.randn(3 * D),
             "decoder.layers.0.self_attn.out_proj.weight": torch.randn(D, D),
             "decoder.layers.0.self_attn.out_proj.bias": torch.randn(D),
             "decoder.layers.0.fc1.weight": torch.randn(F, D), "decoder.layers.0.fc1.bias": torch.randn(F),
             "decoder.layers.0.fc2.weight": torch.randn(D, F), "decoder.layers.0.fc2.bias": torch.randn(D),
             "decoder.layers.0.final_layer_norm.weight": torch.randn(D), "decoder.version": torch.tensor([3.0])}
    four = reshard_megatron_parts([whole], 4)
    assert four[0]["decoder.layers.0.fc1.weight"].shape == (F // 4, D)
    assert four[0]["decoder.layers.0.fc2.weight"].shape == (D, F // 4)
    assert four[1]["decoder.layers.0.self_attn.qkv_proj.weight"].shape == (3 * D // 4, D)
    # part 1 of the fused projection holds rows [2:4] of each of the three blocks
    blocks = whole["decoder.layers.0.self_attn.qkv_proj.weight"].view(3, D, D)
    assert torch.equal(four[1]["decoder.layers.0.self_attn.qkv_proj.weight"], blocks[:, 2:4].reshape(-1, D))
    two = reshard_megatron_parts({i: p for i, p in enumerate(four)}, 2)
    back = reshard_megatron_parts(two, 1)[0]
    assert back.keys() == whole.keys() and all(torch.equal(back[k], whole[k]) for k in whole)
    assert get_n_layers(back) == 1
    assert find_num_parts(["a-model_part-0-shard1.pt", "a-model_part-3-shard0.pt"]) == 4 and find_num_parts(["a.pt"]) == 0


def test_nll_loss_gather_branch_matches_torch(monkeypatch):
    from metaseq_b200.criterions import cross_entropy as ce

    torch.manual_seed(0)
    lp = torch.log_softmax(torch.randn(6, 7), -1)
    tgt = torch.tensor([1, 2, 1, 0, 3, 6])
    want = {r: torch.nn.functional.nll_loss(lp, tgt, ignore_index=1, reduction=r) for r in ("mean", "sum", "none")}
    assert torch.allclose(ce.nll_loss(lp, tgt, ignore_index=1, reduction="sum"), want["sum"])
    monkeypatch.setattr(ce, "_GATHER_ABOVE", 0)  # force the path meant for inputs beyond 2e9 elements
    assert torch.allclose(ce.nll_loss(lp, tgt, ignore_index=1, reduction="sum"), want["sum"])
    assert torch.allclose(ce.nll_loss(lp, tgt, ignore_index=1, reduction="none"), want["none"])
    # "mean" on that path averages over all rows, as the reference's does
    assert torch.allclose(ce.nll_loss(lp, tgt, ignore_index=1, reduction="mean"), want["sum"] / 6)
    assert torch.allclose(ce.nll_loss(lp, tgt, reduction="mean"), torch.nn.functional.nll_loss(lp, tgt))
    with pytest.raises(NotImplementedError):
        ce.nll_loss(lp, tgt, reduction="bogus")


def test_plasma_store_owns_and_unlinks_shared_segments():
    from multiprocessing import shared_memory

    from metaseq_b200.data.plasma_utils import PlasmaStore

    store = PlasmaStore()
    seg = store.register(shared_memory.SharedMemory(create=True, size=64))
    name = seg.name
    store.close()
    with pytest.raises(FileNotFoundError):
        shared_memory.SharedMemory(name=name)
    store.close()  # idempotent


def test_sinusoidal_positions_compile_with_torchscript(tmp_path):
    """The reference exports this module with torch.jit.script (tests/test_export.py): the compiled module must save,
    load and give the eager result, including the growth of its table beyond the initial size."""
    from metaseq_b200.modules.sinusoidal_positional_embedding import SinusoidalPositionalEmbedding

    m = SinusoidalPositionalEmbedding(embedding_dim=8, padding_idx=1, init_size=16)
    scripted = torch.jit.script(m)
    path = str(tmp_path / "pos.pt")
    scripted.save(path)
    loaded = torch.jit.load(path)
    x = torch.tensor([[5, 6, 1, 1], [1, 7, 8, 9]])
    assert torch.equal(loaded(x), m(x))
    assert torch.all(m(x)[0, 2:] == 0)  # padding rows
    long = torch.randint(2, 50, (1, 300))
    assert torch.allclose(loaded(long), m(long))


def test_modules_keep_separate_slots_of_one_incremental_state():
    """Two modules sharing one incremental-state dictionary do not see each other's entries (the reference checks this
    on scripted attention modules: tests/test_export.py:73-91)."""
    from metaseq_b200.incremental_decoding_utils import with_incremental_state

    @with_incremental_state
    class Holder(torch.nn.Module):
        pass

    a, b = Holder(), Holder()
    state = {}
    state = a.set_incremental_state(state, "key", {"a": torch.tensor([1])})
    state = b.set_incremental_state(state, "key", {"a": torch.tensor([2])})
    assert int(a.get_incremental_state(state, "key")["a"]) == 1
    assert int(b.get_incremental_state(state, "key")["a"]) == 2


def test_standalone_scaled_masked_softmax_functions_match_autograd_of_plain_ops():
    from metaseq_b200.modules.fused_softmax import scaled_masked_softmax, scaled_upper_triang_masked_softmax

    torch.manual_seed(0)
    x = torch.randn(6, 5, 5, dtype=torch.double, requires_grad=True)
    y = scaled_upper_triang_masked_softmax(x, 0.3)
    hidden = torch.ones(5, 5, dtype=torch.bool).triu(1)
    ref = torch.softmax((x * 0.3).masked_fill(hidden, float("-inf")), dim=-1)
    assert torch.allclose(y.double(), ref, atol=1e-6)
    assert (y.masked_select(hidden.expand_as(y)) == 0).all()
    w = torch.randn_like(ref)
    (gx,) = torch.autograd.grad((y * w).sum(), x)
    (gr,) = torch.autograd.grad((ref * w).sum(), x)
    assert torch.allclose(gx, gr, atol=1e-6)

    x4 = torch.randn(2, 3, 4, 7, requires_grad=True)
    mask = torch.rand(2, 1, 4, 7) < 0.3
    mask[0, 0, 1] = True  # one fully hidden row: uniform, not NaN
    y4 = scaled_masked_softmax(x4, mask, 0.5)
    ref4 = torch.softmax((x4 * 0.5).masked_fill(mask, -10000.0), dim=-1)
    assert torch.allclose(y4, ref4, atol=1e-6)
    assert torch.allclose(y4[0, :, 1], torch.full((3, 7), 1 / 7), atol=1e-6)
    w4 = torch.randn_like(ref4)
    (g4,) = torch.autograd.grad((y4 * w4).sum(), x4)
    (g4r,) = torch.autograd.grad((ref4 * w4).sum(), x4)
    # the backward pass sees only the probabilities (as the reference's kernel does), so a fully hidden row gets
    # the gradient of a plain softmax where autograd through the fill gives zero; every other row agrees
    keep = torch.ones(2, 3, 4, dtype=torch.bool)
    keep[0, :, 1] = False
    assert torch.allclose(g4[keep], g4r[keep], atol=1e-6)


def test_config_store_lists_registered_components_and_composes_a_root_config():
    import metaseq_b200.criterions  # noqa: F401  (registration side effects)
    import metaseq_b200.models  # noqa: F401
    import metaseq_b200.optim  # noqa: F401
    import metaseq_b200.optim.lr_scheduler  # noqa: F401
    import metaseq_b200.tasks  # noqa: F401
    from metaseq_b200.dataclass.configs import CommonConfig, MetaseqConfig
    from metaseq_b200.dataclass.initialize import ConfigStore, compose, hydra_init

    hydra_init()
    hydra_init()  # idempotent
    cs = ConfigStore.instance()
    assert isinstance(cs.load("base_config"), MetaseqConfig)
    assert isinstance(cs.load("common"), CommonConfig)
    assert {"task", "model", "optimizer", "lr_scheduler", "criterion"} <= set(cs.groups())
    assert "language_modeling" in cs.list("task") and "transformer_lm" in cs.list("model")
    with pytest.raises(KeyError, match="no config named"):
        cs.load("nope", group="task")

    cfg = compose(["common.seed=7", "task=language_modeling", "common.fp16=true", "task.tokens_per_sample=512",
                   "optimization.lr=[0.001]", "lr_scheduler=polynomial_decay"])
    assert cfg.common.seed == 7 and cfg.common.fp16 is True
    assert cfg.task.tokens_per_sample == 512 and cfg.task._name == "language_modeling"
    assert cfg.optimization.lr == [0.001]
    assert cs.load("common").seed != 7  # stored defaults are untouched
    with pytest.raises(KeyError, match="is not set"):
        compose(["optimizer.lr=[0.1]"])
    with pytest.raises(KeyError, match="unknown field"):
        compose(["common.not_a_field=1"])


def test_flat_namespace_round_trips_through_override_strings():
    from typing import Any, Optional

    from metaseq_b200 import options
    from metaseq_b200.dataclass.initialize import compose
    from metaseq_b200.dataclass.utils import convert_namespace_to_config, interpret_dc_type, override_module_args

    argv = ["--task", "dummy_lm", "--dict-size", "124", "--tokens-per-sample", "16", "--batch-size", "2", "--arch",
            "transformer_lm_megatron", "--decoder-layers", "2", "--decoder-embed-dim", "32", "--criterion",
            "cross_entropy", "--optimizer", "adam", "--lr", "1e-2", "--lr-scheduler", "polynomial_decay",
            "--total-num-update", "100", "--clip-norm", "0.5", "--fp16"]
    args = options.parse_args_and_arch(options.get_training_parser(), input_args=argv)
    overrides, deletes = override_module_args(args)
    assert "task=dummy_lm" in overrides and "task._name=dummy_lm" in overrides
    assert "model._name=transformer_lm_megatron" in overrides and "optimization.lr=[0.01]" in overrides
    assert "bpe" in deletes and "tokenizer" in deletes
    cfg, ref = compose(overrides, deletes=deletes), convert_namespace_to_config(args)
    assert cfg.optimization.lr == ref.optimization.lr == [0.01] and cfg.optimization.clip_norm == 0.5
    assert cfg.common.fp16 is True and cfg.task.tokens_per_sample == 16 and cfg.model.decoder_layers == 2
    assert cfg.lr_scheduler.total_num_update == ref.lr_scheduler.total_num_update and cfg.bpe is None
    assert interpret_dc_type(Optional[int]) is int and interpret_dc_type(Any) is str
    with pytest.raises(RuntimeError):
        interpret_dc_type("int")


def test_dense_future_mask_matches_its_compact_form():
    import argparse

    from metaseq_b200.data.dictionary import Dictionary
    from metaseq_b200.models.transformer_decoder import ModelParallelTransformerDecoder
    from metaseq_b200.modules.embedding import Embedding

    def build(**kw):
        args = argparse.Namespace(decoder_embed_dim=16, decoder_attention_heads=2, decoder_ffn_embed_dim=32,
                                  decoder_layers=1, dropout=0.0, attention_dropout=0.0, activation_fn="relu",
                                  tokens_per_sample=8, max_target_positions=8, decoder_learned_pos=True,
                                  share_decoder_input_output_embed=True, **kw)
        d = Dictionary.synthetic(24)
        return ModelParallelTransformerDecoder(args, d, Embedding(len(d), 16, d.pad()))

    x = torch.zeros(5, 2, 16)  # [T, B, C]
    causal = build().buffered_future_mask(x)
    assert causal.shape == (5, 5) and torch.equal(causal == 0, torch.ones(5, 5).tril().bool())
    toks = torch.tensor([[5, 6, 2, 7, 8], [5, 6, 7, 8, 9]])
    docs = build(self_attn_doc_sep=2).buffered_future_mask(x, toks)
    assert docs.shape == (2, 5, 5)
    assert torch.isinf(docs[0, 3, :3]).all() and (docs[0, 3, 3] == 0) and (docs[0, 2, :3] == 0).all()
    assert torch.equal(docs[1], causal)
    ali = build(alibi=True).buffered_future_mask(x)
    assert ali.shape == (4, 5, 5) and torch.isinf(ali[0, 0, 1]) and ali[0, 4, 3] > ali[0, 4, 2] > ali[0, 4, 1]


def test_base_model_takes_its_decoder_in_the_constructor_and_checks_its_type():
    from metaseq_b200.models.base_decoder import BaseDecoder
    from metaseq_b200.models.base_model import BaseModel, check_type

    class Dec(BaseDecoder):
        def __init__(self):
            super().__init__(dictionary=None)

        def forward(self, tokens, **kw):
            return tokens.float().unsqueeze(-1), {"inner_states": []}

        def max_positions(self):
            return 77

    class Wrapper(torch.nn.Module):  # what a sharding wrapper looks like from outside
        def __init__(self, inner):
            super().__init__()
            self.unwrapped_module = inner

    class MyLM(BaseModel):
        def __init__(self, decoder):
            super().__init__(decoder)

    m = MyLM(Dec())
    assert m.max_positions() == 77 and m.max_decoder_positions() == 77 and m.supported_targets == {"future"}
    assert m(torch.tensor([[1, 2]]))[0].shape == (1, 2, 1)
    assert m.eval() is m
    check_type(Wrapper(Dec()), BaseDecoder)
    with pytest.raises(AssertionError):
        MyLM(torch.nn.Linear(2, 2))
    with pytest.raises(NotImplementedError):
        MyLM.from_pretrained("anything")
    assert MyLM.hub_models() == {}


def test_generator_interface_text_codec_normalises_line_ends():
    from metaseq_b200.hub_utils import GeneratorInterface

    class Tok:
        def encode(self, text):
            import types

            assert "\r" not in text
            return types.SimpleNamespace(ids=[ord(c) for c in text])

        def decode(self, ids):
            return "".join(chr(i) for i in ids)

    gi = GeneratorInterface.__new__(GeneratorInterface)
    import types

    gi.bpe = types.SimpleNamespace(bpe=Tok())
    ids = gi.encode_fn("a\r\nb\rc")
    assert gi.decode_fn(ids) == "a\nb\nc"


def test_dataset_protocol_extras_batch_shapes_member_attributes_and_per_dataset_order():
    from metaseq_b200.data.concat_dataset import ConcatDataset
    from metaseq_b200.data.token_transforms import ListDataset

    from metaseq_b200.data.base_dataset import BaseDataset

    sizes = np.array([1, 2, 5, 2, 1, 4, 2])

    class Shaped(BaseDataset):
        def __len__(self):
            return len(sizes)

        def __getitem__(self, i):
            return list(range(sizes[i]))

        def num_tokens(self, i):
            return int(sizes[i])

        def num_tokens_vec(self, indices):
            return sizes[indices]

        def get_batch_shapes(self):
            return [(4, 2), (None, 5)]  # up to 4 samples of <= 2 tokens, or as many of <= 5 as the token budget allows

    ds = Shaped()
    batches = ds.batch_by_size(np.argsort(sizes, kind="stable"), max_tokens=10)
    assert sorted(i for b in batches for i in b) == list(range(len(sizes)))
    for b in batches:
        longest = max(sizes[i] for i in b)
        assert (len(b) <= 4 and longest <= 2) or (len(b) <= 2 and longest <= 5)
    assert ListDataset([1], np.array([1])).get_batch_shapes() is None

    class Plain(BaseDataset):
        def __init__(self, items, tag):
            super().__init__()
            self.items, self.tag = items, tag
            self.sizes = np.array([len(x) for x in items])

        def __len__(self):
            return len(self.items)

        def __getitem__(self, i):
            return self.items[i]

        def size(self, i):
            return int(self.sizes[i])

        def ordered_indices(self):
            return np.argsort(self.sizes, kind="stable")

    a, b = Plain([[1], [2, 2]], "first"), Plain([[3, 3, 3]], "second")
    cat = ConcatDataset([a, b])
    assert cat.attr("tag", 0) == "first" and cat.attr("tag", 2) == "second" and cat.attr("missing", 2) is None
    per = cat.ordered_indices_per_dataset()
    assert [p.tolist() for p in per] == [[0, 1], [2]]


def test_service_queue_keys_hashing_and_the_blocking_worker_entry():
    import queue
    import threading

    from metaseq_b200.service.queue import PriorityQueueRingShard
    from metaseq_b200.service.workers import WorkItem

    key = PriorityQueueRingShard.key_from_dictionary({"top_p": 0.9, "n": 1})
    assert key == "n:1:top_p:0.9"
    idx = PriorityQueueRingShard.get_shard_index_for_key(key, num_shards=8)
    assert idx == PriorityQueueRingShard.get_shard_index_for_key(key, num_shards=8) and 0 <= idx < 8
    assert PriorityQueueRingShard.get_shard_index_for_key(key, num_shards=1) == 0

    batch_queue = queue.PriorityQueue()

    def serve():
        item = batch_queue.get()
        assert item.cost == 25 + 7 and item.data["input"] == list(range(25)) and item.data["temperature"] == 0.5
        item.return_queue.put((item.uid, {"text": "done"}))

    threading.Thread(target=serve, daemon=True).start()
    assert WorkItem.generate_worker(list(range(25)), batch_queue, temperature=0.5) == {"text": "done"}


def test_nan_detector_watches_added_modules_and_names_the_first_bad_one(caplog):
    from metaseq_b200.nan_detector import NanDetector

    class Bad(torch.nn.Module):
        def forward(self, x):
            return x / 0.0

    net = torch.nn.Sequential(torch.nn.Linear(4, 4), Bad())
    extra = Bad()
    with caplog.at_level("WARNING"):
        with NanDetector(net, backward=False) as det:
            det.add_hooks(extra)
            net(torch.ones(2, 4))
            det.reset()
            extra(torch.ones(2, 4))
    assert caplog.text.count("detected in output of") == 2 and "forward" in caplog.text


def test_shared_memory_array_publishes_once_and_reattaches_after_pickling():
    from metaseq_b200.data.plasma_utils import PlasmaArray

    small = PlasmaArray(np.arange(10))
    assert small.plasma is None and small.client is None
    big = PlasmaArray(np.arange(400_000, dtype=np.int64))
    assert big.plasma is not None and big.client is None
    big.start_server()
    name = big.client.name
    big.start_server()
    assert big.client.name == name
    clone = pickle.loads(pickle.dumps(big))
    assert clone.client.name == name and int(clone.array[-1]) == 399_999


def test_packages_export_the_names_that_reference_code_imports_from_them():
    import importlib

    wanted = {
        "modules": ["ActivationFn", "Dropout", "FeedForward", "LayerNorm", "LayerNormFp32", "LearnedPositionalEmbedding",
                    "Linear", "ModelParallelMultiheadAttention", "ModelParallelTransformerDecoderLayer",
                    "PositionalEmbedding", "SinusoidalPositionalEmbedding", "gelu", "AdaptiveSoftmax"],
        "data": ["CountingIterator", "EpochBatchIterator", "GroupedIterator", "ShardedIterator", "MultiplePadDataset",
                 "Dictionary", "JsonlDataset", "MonolingualDataset", "TokenBlockDataset"],
        "models": ["DistributedModel", "BaseModel", "BaseDecoder", "IncrementalDecoder"],
        "optim": ["LegacyOptimizer", "shard_", "FP16Optimizer", "MemoryEfficientFP16Optimizer", "BaseOptimizer"],
    }
    for pkg, names in wanted.items():
        module = importlib.import_module("metaseq_b200." + pkg)
        for name in names:
            assert getattr(module, name) is not None, (pkg, name)
        assert set(names) <= set(dir(module))
    with pytest.raises(AttributeError):
        importlib.import_module("metaseq_b200.modules").NoSuchLayer


def test_distributed_import_path_of_the_reference_resolves_to_the_parallel_package():
    import metaseq_b200.distributed.utils as by_path
    import metaseq_b200.parallel.utils as real
    from metaseq_b200.distributed import FullyShardedDataParallel, ModuleProxyWrapper, fsdp_enable_wrap, fsdp_wrap  # noqa: F401
    from metaseq_b200.distributed import utils as distributed_utils
    from metaseq_b200.distributed.rendezvous import ComplicitStore  # noqa: F401
    from metaseq_b200.distributed.stitch_fsdp_ckpt import consolidate_fsdp_shards, reshard_megatron_parts  # noqa: F401

    assert by_path is real and distributed_utils is real
    assert distributed_utils.get_global_world_size() == 1
