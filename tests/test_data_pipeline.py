"""Data pipeline on CPU: dictionary, JSONL datasets, document -> sequence packing, streaming iterator resume,
partitioning, token blocks (native vs Python), batching (native vs Python), binary datasets, CM3 objective."""
import json
import os

import numpy as np
import pytest
import torch

from metaseq_b200.data import (
    CausalMaskedDocumentToSequenceDataset,
    Dictionary,
    DocumentToSequenceDataset,
    JsonlDataset,
    PartitionedStreamingDataset,
    StreamingShuffleDataset,
    StreamingTokenBlockDataset,
    TokenBlockDataset,
    data_utils,
)
from metaseq_b200.data import indexed_dataset, iterators
from metaseq_b200.data.token_block_dataset import get_block_to_dataset_index, get_slice_indices, get_slice_indices_py


class TensorListDataset(torch.utils.data.Dataset):
    def __init__(self, items):
        self.items = items
        self.sizes = np.array([len(x) for x in items])

    def __getitem__(self, i):
        return self.items[i]

    def __len__(self):
        return len(self.items)


def _docs(n=40, seed=0, lo=3, hi=30):
    rng = np.random.RandomState(seed)
    return [torch.arange(100 * i, 100 * i + rng.randint(lo, hi)) for i in range(n)]


def test_dictionary_special_symbols_and_roundtrip(tmp_path):
    d = Dictionary()
    assert (d.bos(), d.pad(), d.eos(), d.unk()) == (0, 1, 2, 3)
    for w in ["hello", "world", "hello"]:
        d.add_symbol(w)
    assert len(d) == 6 and d.index("hello") == 4 and d.index("nope") == d.unk()
    d.save(str(tmp_path / "dict.txt"))
    d2 = Dictionary.load(str(tmp_path / "dict.txt"))
    assert d2.symbols == d.symbols
    d2.pad_to_multiple_(8)
    assert len(d2) % 8 == 0


def test_jsonl_dataset_index_cache_and_subshards(tmp_path):
    path = tmp_path / "data.jsonl"
    with open(path, "w") as f:
        for i in range(23):
            f.write(json.dumps({"text": f"doc {i}"}) + "\n")
    ds = JsonlDataset(str(path), tokenizer=lambda obj: obj["text"])
    assert len(ds) == 23 and ds[5] == "doc 5"
    assert os.path.exists(str(path) + ".fairseq.idx.npy")
    # a corrupted index cache is rebuilt, not trusted
    with open(str(path) + ".fairseq.idx.npy", "wb") as f:
        f.write(b"garbage")
    ds = JsonlDataset(str(path), tokenizer=lambda obj: obj["text"], recache=True)
    assert len(ds) == 23
    seen = []
    for epoch in range(1, 4):
        sub = JsonlDataset(str(path), tokenizer=lambda obj: obj["text"], epoch=epoch, data_subshard_count=3)
        seen += [sub[i] for i in range(len(sub))]
    assert sorted(seen) == sorted(f"doc {i}" for i in range(23))


@pytest.mark.parametrize("break_mode", ["none", "complete", "eos_pad_8"])
def test_document_to_sequence_covers_every_token(break_mode):
    docs = _docs()
    ds = DocumentToSequenceDataset(TensorListDataset(docs), block_size=32, break_mode=break_mode, drop_last=False,
                                   padding_idx=-1, seed=1, permute_documents=False)
    ds.set_epoch(1)
    blocks = list(ds)
    got = torch.cat([b["block"][b["block"] != -1] for b in blocks])
    want = torch.cat([d[:32] if break_mode == "eos_pad_8" else d for d in docs])
    assert torch.equal(torch.sort(got).values, torch.sort(want).values)
    for b in blocks:
        if break_mode == "eos_pad_8":
            assert len(b["block"]) % 8 == 0 and len(b["block"]) <= 32
        else:
            assert len(b["block"]) == 32


def test_document_to_sequence_epoch_permutation_is_deterministic():
    docs = _docs()

    def run(epoch):
        ds = DocumentToSequenceDataset(TensorListDataset(docs), 16, "none", drop_last=True, padding_idx=1, seed=7,
                                       shuffle_buffer_size=5)
        ds.set_epoch(epoch)
        return [b["block"].tolist() for b in ds]

    assert run(1) == run(1)
    assert run(1) != run(2)


def test_to_skip_equals_dropping_a_prefix():
    docs = _docs()
    full = DocumentToSequenceDataset(TensorListDataset(docs), 16, "none", drop_last=True, padding_idx=1, seed=3)
    full.set_epoch(1)
    all_blocks = [b["block"].tolist() for b in full]
    part = DocumentToSequenceDataset(TensorListDataset(docs), 16, "none", drop_last=True, padding_idx=1, seed=3, to_skip=5)
    part.set_epoch(1)
    assert [b["block"].tolist() for b in part] == all_blocks[5:]


def _make_iterator(docs, num_workers=0, epoch=1):
    ds = DocumentToSequenceDataset(TensorListDataset(docs), 16, "none", drop_last=True, padding_idx=1, seed=5,
                                   shuffle_buffer_size=4)
    ds.set_epoch(epoch)
    return iterators.StreamingEpochBatchIterator(
        ds, batch_size=3, collate_fn=lambda items: torch.stack([x["block"] for x in items]), drop_last=True,
        num_workers=num_workers, epoch=epoch)


def test_streaming_iterator_resumes_mid_epoch():
    docs = _docs(80)
    ref_itr = _make_iterator(docs)
    reference = [b.tolist() for b in ref_itr.next_epoch_itr()]
    assert len(reference) > 6
    itr = _make_iterator(docs)
    epoch_itr = itr.next_epoch_itr()
    first = [next(epoch_itr).tolist() for _ in range(4)]
    state = itr.state_dict()
    resumed = _make_iterator(docs)
    resumed.load_state_dict(state)
    rest = [b.tolist() for b in resumed.next_epoch_itr()]
    assert first + rest == reference
    # a second interruption, from the resumed iterator
    again = _make_iterator(docs)
    again.load_state_dict(state)
    it2 = again.next_epoch_itr()
    two = [next(it2).tolist() for _ in range(2)]
    state2 = again.state_dict()
    third = _make_iterator(docs)
    third.load_state_dict(state2)
    assert first + two + [b.tolist() for b in third.next_epoch_itr()] == reference


def test_partitioned_streaming_dataset_round_robin():
    items = list(range(10))

    class It(torch.utils.data.IterableDataset):
        def __iter__(self):
            return iter(items)

    parts = [list(PartitionedStreamingDataset(It(), num_shards=3, shard_id=r, drop_last=False)) for r in range(3)]
    assert parts[0][:4] == [0, 3, 6, 9]
    assert len(parts[0]) == len(parts[1]) == len(parts[2])  # padded with None to equal length
    assert [x for x in parts[1] if x is not None] == [1, 4, 7]
    dropped = [list(PartitionedStreamingDataset(It(), num_shards=3, shard_id=r, drop_last=True)) for r in range(3)]
    assert all(len(p) == 3 for p in dropped)


def test_streaming_shuffle_dataset_is_a_seeded_permutation():
    base = TensorListDataset([torch.tensor([i]) for i in range(20)])
    ds = StreamingShuffleDataset(base, seed=11)
    ds.set_epoch(1)
    a = [int(x) for x in ds]
    ds.set_epoch(1)
    assert a == [int(x) for x in ds]
    ds.set_epoch(2)
    b = [int(x) for x in ds]
    assert sorted(a) == list(range(20)) == sorted(b) and a != b


@pytest.mark.parametrize("mode", ["none", "complete", "complete_doc", "eos"])
def test_token_block_slices_native_matches_python(mode):
    rng = np.random.RandomState(4)
    sizes = rng.randint(1, 40, size=200).astype(np.int64)
    sizes[::17] = 1  # document separators for complete_doc
    a = get_slice_indices(sizes, mode, 64)
    b = get_slice_indices_py(sizes, mode, 64)
    assert a.tolist() == b.tolist()
    idx = get_block_to_dataset_index(sizes, a)
    cum = np.concatenate([[0], np.cumsum(sizes)])
    for (s, e), (first, off, last) in zip(a, idx):
        assert cum[first] + off == s and cum[last] < e <= cum[last + 1]


def test_token_block_dataset_items_and_targets():
    docs = [torch.arange(1, 6), torch.arange(10, 13), torch.arange(20, 30)]
    base = TensorListDataset(docs)
    ds = TokenBlockDataset(base, base.sizes, block_size=6, pad=0, eos=2, break_mode="none", include_targets=True)
    flat = torch.cat(docs)
    assert torch.equal(torch.cat([ds[i][1] for i in range(len(ds))]), flat)
    src, tgt, past = ds[1]
    assert torch.equal(src, flat[5:11]) and torch.equal(tgt, flat[6:12])
    # the block starts one token into its first item: history before that item is replaced by eos
    assert past.tolist() == [2] + flat[5:10].tolist()
    src0, tgt0, _ = ds[0]
    assert src0[0] == 2 and torch.equal(src0[1:], tgt0[:-1])


def test_batch_fixed_shapes_native_matches_python():
    rng = np.random.RandomState(3)
    shapes = np.array([[16, 8], [8, 16], [4, 32], [2, 64]], dtype=np.int64)
    sizes = rng.randint(1, 70, size=400).astype(np.int64)
    idx = rng.permutation(400).astype(np.int64)
    a = data_utils.batch_by_size(idx, num_tokens_vec=sizes[idx], fixed_shapes=shapes)
    b = data_utils.batch_fixed_shapes_py(idx, sizes[idx], shapes.tolist())
    assert a == b
    assert [i for batch in a for i in batch] == idx.tolist()  # order kept, nothing dropped
    for batch in a:
        longest = int(max(sizes[batch]))
        assert any(len(batch) <= r and longest <= t for r, t in shapes) or (len(batch) == 1 and longest > 64)
    # the size-callback form is the vector form
    c = data_utils.batch_by_size_fn(idx, lambda i: int(sizes[i]), max_tokens=128, max_sentences=9)
    d = data_utils.batch_by_size(idx, num_tokens_vec=sizes[idx], max_tokens=128, max_sentences=9)
    assert c == d


def test_batch_by_size_native_matches_python():
    rng = np.random.RandomState(0)
    for max_tokens, max_sent, mult in [(100, None, 1), (64, 5, 1), (256, 16, 8), (None, 7, 1)]:
        sizes = rng.randint(1, 60, size=500).astype(np.int64)
        idx = np.argsort(sizes, kind="mergesort")
        a = data_utils.batch_by_size(idx, num_tokens_vec=sizes[idx], max_tokens=max_tokens, max_sentences=max_sent,
                                     required_batch_size_multiple=mult)
        b = data_utils.batch_by_size_py(idx, sizes[idx], max_tokens if max_tokens is not None else -1,
                                        max_sent if max_sent is not None else -1, mult)
        assert [list(x) for x in a] == [list(x) for x in b]
        assert sorted(i for batch in a for i in batch) == sorted(idx.tolist())
        for batch in a:
            if max_tokens is not None:
                assert len(batch) * max(sizes[batch]) <= max_tokens or len(batch) == 1
            if max_sent is not None:
                assert len(batch) <= max_sent


@pytest.mark.parametrize("impl", ["mmap", "lazy"])
def test_indexed_dataset_roundtrip_and_merge(tmp_path, impl):
    items = [torch.arange(5), torch.tensor([7, 8]), torch.arange(100, 120)]
    prefix = str(tmp_path / impl)
    b = indexed_dataset.make_builder(prefix + ".bin", impl, vocab_size=50000)
    for t in items:
        b.add_item(t)
    b.finalize(prefix + ".idx")
    ds = indexed_dataset.make_dataset(prefix, "mmap" if impl == "mmap" else "cached", fix_lua_indexing=True)
    assert len(ds) == 3 and all(torch.equal(ds[i], items[i]) for i in range(3))
    assert list(ds.sizes) == [5, 2, 20]
    assert indexed_dataset.infer_dataset_impl(prefix) == ("mmap" if impl == "mmap" else "cached")
    prefix2 = str(tmp_path / (impl + "_merged"))
    b2 = indexed_dataset.make_builder(prefix2 + ".bin", impl, vocab_size=50000)
    b2.add_item(torch.tensor([1, 2, 3]))
    b2.merge_file_(prefix)
    b2.finalize(prefix2 + ".idx")
    merged = indexed_dataset.make_dataset(prefix2, "mmap" if impl == "mmap" else "lazy", fix_lua_indexing=True)
    assert len(merged) == 4 and torch.equal(merged[3], items[2]) and torch.equal(merged[0], torch.tensor([1, 2, 3]))


def test_streaming_token_block_dataset_modes():
    docs = [torch.arange(1, n + 1) for n in (5, 12, 3, 9)]
    none = [b["block"].tolist() for b in StreamingTokenBlockDataset(docs, 8, "none", padding_idx=0)]
    assert none[0] == [1, 2, 3, 4, 5, 1, 2, 3] and all(len(b) == 8 for b in none)
    assert sum(x != 0 for b in none for x in b) == 29
    complete = [b["block"].tolist() for b in StreamingTokenBlockDataset(docs, 8, "complete", padding_idx=0)]
    assert complete[0] == [1, 2, 3, 4, 5, 0, 0, 0]
    with pytest.raises(ValueError):
        StreamingTokenBlockDataset(docs, 8, "bogus", padding_idx=0)


def test_cm3_objective_moves_spans_behind_sentinels():
    torch.manual_seed(0)
    np.random.seed(0)
    doc = torch.arange(10, 60)
    ds = CausalMaskedDocumentToSequenceDataset(
        sentinel_token_expectation=1, sentinel_tokens=[1000], sentinel_method="fixed", sentinel_eos=999,
        allow_rotation_across_eod=True, eod=2, dataset=TensorListDataset([doc]), block_size=50, break_mode="none",
        drop_last=False, padding_idx=1, seed=1, permute_documents=False)
    ds.set_epoch(1)
    toks = next(iter(ds))["block"].tolist()
    assert len(toks) <= 50 and toks.count(1000) in (1, 2)
    first = toks.index(1000)
    assert toks[:first] == doc[:first].tolist()  # the prefix before the cut is untouched
    if toks.count(1000) == 2:
        second = toks.index(1000, first + 1)
        tail = toks[second + 1:]
        span = tail[:tail.index(999)] if 999 in tail else tail
        # the span removed at the first sentinel reappears, in order, after the second one
        assert span == list(range(10 + first, 10 + first + len(span)))
        # and the text between the sentinels continues after the removed span
        middle = toks[first + 1:second]
        assert middle == list(range(middle[0], middle[0] + len(middle))) if middle else True


def test_monolingual_dataset_clips_targets_and_prepends_language_ids():
    from metaseq_b200.data.dictionary import Dictionary
    from metaseq_b200.data.monolingual_dataset import MonolingualDataset

    src_vocab, tgt_vocab = Dictionary(), Dictionary()
    for i in range(20):
        src_vocab.add_symbol(f"w{i}")
    for i in range(8):
        tgt_vocab.add_symbol(f"w{i}")
    n_tgt = len(tgt_vocab)
    blocks = [(torch.tensor([5, 6, 7]), torch.tensor([6, 7, n_tgt + 3]), torch.tensor([4, 5, 6])),
              (torch.tensor([9, 10]), torch.tensor([10, n_tgt]), torch.tensor([8, 9]))]
    ds = MonolingualDataset(blocks, [3, 2], src_vocab, tgt_vocab, add_bos_token=True, src_lang_idx=17, tgt_lang_idx=6)
    item = ds[0]
    assert item["source"].tolist() == [17, 5, 6, 7]
    assert item["target"].tolist() == [6, 6, 7, tgt_vocab.unk()]
    assert blocks[0][1].tolist() == [6, 7, n_tgt + 3]  # the wrapped dataset's tensors are left alone
    batch = ds.collater([ds[0], ds[1]])
    assert batch["net_input"]["src_tokens"].tolist() == [[17, 5, 6, 7], [17, 9, 10, src_vocab.pad()]]
    assert batch["target"][1].tolist() == [6, 10 if 10 < n_tgt else tgt_vocab.unk(), tgt_vocab.unk(), src_vocab.pad()]
    assert batch["ntokens"] == 7 and batch["net_input"]["src_lengths"].tolist() == [4, 3]
    plain = MonolingualDataset(blocks, [3, 2], src_vocab, add_bos_token=True)
    assert plain[1]["source"].tolist() == [src_vocab.bos(), 9, 10] and plain[1]["target"].tolist()[0] == src_vocab.bos()
    assert plain.ordered_indices().tolist() == [1, 0]
