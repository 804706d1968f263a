"""Resampling wrapper and context-window evaluation wrapper (the behaviours that the reference pins in
tests/test_resampling_dataset.py and tests/test_lm_context_window.py)."""
import collections
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from metaseq_b200.data.dictionary import Dictionary
from metaseq_b200.data.monolingual_dataset import MonolingualDataset
from metaseq_b200.data.resampling_dataset import ResamplingDataset
from metaseq_b200.data.token_transforms import ListDataset
from metaseq_b200.tasks.language_modeling import LanguageModelingTask


STRINGS = ["ab", "c", "def", "ghij"]
WEIGHTS = [4.0, 2.0, 7.0, 1.5]


def _resampled(**kw):
    base = ListDataset(STRINGS, np.array([len(s) for s in STRINGS]))
    return ResamplingDataset(base, **kw)


@pytest.mark.parametrize("batch_by_size", [True, False])
def test_resampling_length_stability_sizes_and_order(batch_by_size):
    ds = _resampled(weights=WEIGHTS, size_ratio=2, batch_by_size=batch_by_size, seed=3)
    assert len(ds) == 2 * len(STRINGS)
    first = [ds[i] for i in range(len(ds))]
    assert first == [ds[i] for i in range(len(ds))]  # one epoch draws once
    for i, item in enumerate(first):
        assert ds.size(i) == len(item) == ds.num_tokens(i)
    order = list(ds.ordered_indices())
    assert sorted(order) == list(range(len(ds)))
    by_size = [ds.size(i) for i in order]
    if batch_by_size:
        assert by_size == sorted(by_size)
    else:
        assert order == list(range(len(ds)))


def test_resampling_redraws_per_epoch_and_follows_the_weights():
    ds = _resampled(weights=WEIGHTS, size_ratio=2, seed=0)
    counts = collections.Counter()
    draws = set()
    epochs = 1000
    for epoch in range(1, epochs + 1):
        ds.set_epoch(epoch)
        items = tuple(ds[i] for i in range(len(ds)))
        draws.add(items)
        counts.update(items)
    assert len(draws) > epochs // 2  # epochs differ from one another
    total = sum(counts.values())
    assert total == epochs * len(ds)
    for s, w in zip(STRINGS, WEIGHTS):
        assert abs(counts[s] / total - w / sum(WEIGHTS)) < 0.02
    # the same (seed, epoch) gives the same draw in a fresh wrapper
    again = _resampled(weights=WEIGHTS, size_ratio=2, seed=0)
    again.set_epoch(epochs)
    assert tuple(again[i] for i in range(len(again))) == items


def test_resampling_without_weights_is_uniform_and_without_replacement_is_a_permutation():
    ds = _resampled(weights=None, replace=False, size_ratio=1.0, seed=5)
    assert sorted(ds[i] for i in range(len(ds))) == sorted(STRINGS)


def test_context_window_carries_the_corpus_tail_and_masks_its_targets():
    d = Dictionary()
    for i in range(10):
        d.add_symbol(str(i))
    assert len(d) == 14 and d.pad() == 1
    rows = [torch.tensor([4, 5, 6, 7]), torch.tensor([8, 9, 10, 11]), torch.tensor([12, 13])]
    base = ListDataset(rows, np.array([4, 4, 2]))
    mono = MonolingualDataset(base, sizes=np.array([4, 4, 2]), src_vocab=d)
    task = LanguageModelingTask(SimpleNamespace(tokens_per_sample=4, seed=1), d)
    it = task.eval_lm_dataloader(dataset=mono, batch_size=1, context_window=2)

    b = next(it)
    assert b["net_input"]["src_tokens"][0].tolist() == [4, 5, 6, 7, 1, 1]
    assert b["target"][0].tolist() == [4, 5, 6, 7, 1, 1]
    assert b["start_indices"] == [0]
    b = next(it)
    assert b["net_input"]["src_tokens"][0].tolist() == [6, 7, 8, 9, 10, 11]
    assert b["target"][0].tolist() == [1, 1, 8, 9, 10, 11]
    assert b["start_indices"] == [2]
    b = next(it)
    assert b["net_input"]["src_tokens"][0].tolist() == [10, 11, 12, 13]
    assert b["target"][0].tolist() == [1, 1, 12, 13]
    with pytest.raises(StopIteration):
        next(it)


def test_eval_dataloader_without_context_window_is_the_plain_corpus():
    d = Dictionary()
    for i in range(10):
        d.add_symbol(str(i))
    rows = [torch.tensor([4, 5, 6, 7]), torch.tensor([8, 9, 10, 11])]
    mono = MonolingualDataset(ListDataset(rows, np.array([4, 4])), sizes=np.array([4, 4]), src_vocab=d)
    task = LanguageModelingTask(SimpleNamespace(tokens_per_sample=4, seed=1), d)
    batches = list(task.eval_lm_dataloader(dataset=mono, batch_size=2))
    assert len(batches) == 1
    assert batches[0]["net_input"]["src_tokens"].tolist() == [[4, 5, 6, 7], [8, 9, 10, 11]]
