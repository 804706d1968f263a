"""Causal-masked ("CM3") objective on top of ``DocumentToSequenceDataset``: spans of each packed block are
cut out, replaced by sentinel tokens and appended at the end as ``<sentinel> span <eos>`` so that a
left-to-right model learns to infill (reference: metaseq/data/cm3_dataset.py:59-229)."""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch

from .document_to_sequence import DocumentToSequenceDataset

Span = Tuple[int, int]


def span_intersection(left: Span, right: Span) -> bool:
    return max(left[0], right[0]) < min(left[1], right[1])


def overlaps(a: Span, b: Span) -> bool:
    return not (a[1] <= b[0] or a[0] >= b[1])


def calculate_overlap(a: Span, b: Span) -> int:
    return max(0, min(a[1], b[1]) - max(a[0], b[0]))


def adjust_span(span: Span, container: Span) -> Span:
    """Clips ``span`` to ``container``."""
    return (max(span[0], container[0]), min(span[1], container[1]))


def adjust_spans(spans: List[Span], constraints: List[Span]) -> List[Span]:
    """Clips every span to the constraint it overlaps most (so no span crosses a document boundary)."""
    out = []
    for sp in spans:
        best, best_ov = None, 0
        for c in constraints:
            ov = calculate_overlap(sp, c)
            if ov > best_ov:
                best, best_ov = c, ov
        if best is not None and overlaps(sp, best):
            sp = adjust_span(sp, best)
        out.append(sp)
    return out


class CausalMaskedDocumentToSequenceDataset(DocumentToSequenceDataset):
    def __init__(self, sentinel_token_expectation: int, sentinel_tokens: List[int], sentinel_method: str,
                 sentinel_eos: int, allow_rotation_across_eod: bool, eod: int, dataset, block_size: int,
                 break_mode: str = "none", drop_last: Optional[bool] = True, padding_idx: Optional[int] = None,
                 shuffle_buffer_size: int = 1, seed: Optional[int] = None, len_cache=None, to_skip=0,
                 permute_documents=True, source_target=False):
        super().__init__(dataset, block_size, break_mode, drop_last, padding_idx, shuffle_buffer_size, seed, len_cache,
                         to_skip, permute_documents, source_target)
        assert sentinel_method in ("fixed", "poisson"), sentinel_method
        assert len(sentinel_tokens) >= 1
        assert block_size > 1
        assert not source_target, "CM3 objective is not supported when source_target is True"
        self.sentinel_token_expectation = sentinel_token_expectation
        self.sentinel_tokens = sentinel_tokens
        self.sentinel_method = sentinel_method
        self.sentinel_fixed = sentinel_method == "fixed"
        self.tokens_per_sample = block_size
        self.eos = sentinel_eos
        self.allow_rotation_across_eod = allow_rotation_across_eod
        self.eod = eod

    def get_sentinel(self, i):
        return self.sentinel_tokens[i]

    def sentinel_masking(self, document: torch.Tensor, spans: List[Span]):
        doc = document.clone()
        keep = torch.ones_like(doc, dtype=torch.bool)
        for i, (s, e) in enumerate(spans):
            doc[s] = self.get_sentinel(i)
            keep[s + 1:e] = False
        return doc[keep]

    def sentinel_targets(self, document: torch.Tensor, spans: List[Span]):
        if self.sentinel_fixed:
            assert len(self.sentinel_tokens) == len(spans)
        else:
            assert len(self.sentinel_tokens) > len(spans)
        parts = []
        for i, (s, e) in enumerate(spans):
            parts.append(document.new_tensor([self.get_sentinel(i)]))
            parts.append(document[s:e])
            parts.append(document.new_tensor([self.eos]))
        return torch.cat(parts) if parts else document.new_zeros(0)

    def get_spans_to_mask(self, document_length: int) -> Optional[List[Span]]:
        if self.sentinel_fixed:
            n = self.sentinel_token_expectation
        else:
            n = int(torch.poisson(torch.tensor([float(self.sentinel_token_expectation)]))
                    .clamp(0, len(self.sentinel_tokens) - 1).item())
        if n == 0:
            return None
        if n == 1:
            start, end = np.random.uniform(size=2)
            if end < start:
                start, end = end, start
            start = int(start * document_length)
            end = int(end * document_length + 0.5)
            return None if start == end else [(start, end)]
        candidates = [tuple(np.random.uniform(size=2)) for _ in range(n ** 2)]
        candidates = [(int(a * document_length), int(b * document_length + 0.5)) for a, b in candidates]
        candidates = [(a, b) if a <= b else (b, a) for a, b in candidates]
        chosen: List[Span] = []
        while len(chosen) < n and candidates:
            c = candidates.pop()
            if not any(span_intersection(x, c) for x in chosen):
                chosen.append(c)
        return chosen

    def get_ordered_spans(self, spans: List[Span]) -> List[Span]:
        return sorted(spans, key=lambda x: x[0])

    def get_document_boundaries(self, item: torch.Tensor) -> List[Span]:
        bounds = (item == self.eod).nonzero().reshape(-1).tolist()
        if not bounds or bounds[0] != 0:
            bounds = [0] + bounds
        if bounds[-1] != item.size(0) - 1:
            bounds = bounds + [item.size(0)]
        return [(bounds[i - 1], bounds[i]) for i in range(1, len(bounds))]

    def __iter__(self):
        for packed in super().__iter__():
            item = packed["block"]
            assert len(item) > 0
            spans = self.get_spans_to_mask(len(item))
            if spans is not None and not self.allow_rotation_across_eod:
                spans = adjust_spans(spans, self.get_document_boundaries(item))
            if spans is None:
                yield packed
                continue
            spans = self.get_ordered_spans(spans)
            source = self.sentinel_masking(item, spans)
            targets = self.sentinel_targets(item, spans)
            # the sentinel / end-of-span tokens can push the result a token or two past the block size
            packed["block"] = torch.cat([source, targets])[: self.tokens_per_sample]
            yield packed


# --------------------------------------------------------------------- task-side helpers
CM3_END_OF_SPAN = "<eoss>"


def sentinel_names(n: int) -> List[str]:
    """Special tokens the tokenizer needs for the objective: ``n`` span sentinels and the end-of-span marker."""
    return [f"<sentinel:{i}>" for i in range(n)] + [CM3_END_OF_SPAN]


def wrap_cm3(d2s: DocumentToSequenceDataset, task, args) -> CausalMaskedDocumentToSequenceDataset:
    """Rebuilds a plain packed-block dataset as its causal-masked variant using the task's tokenizer ids
    (reference wiring: metaseq/tasks/streaming_language_modeling.py:212-259,400-446)."""
    n = int(args.cm3_num_sentinel_tokens)
    lam = int(args.cm3_lambda_sentinel_tokens)
    assert n > 0, "cm3_num_sentinel_tokens must be > 0"
    assert lam > 0, "cm3_lambda_sentinel_tokens must be > 0"
    assert n >= lam, "cm3_num_sentinel_tokens must be >= cm3_lambda_sentinel_tokens"
    ids = [task.tokenizer.token_to_id(name) for name in sentinel_names(n)[:-1]]
    end = task.tokenizer.token_to_id(CM3_END_OF_SPAN)
    assert all(i is not None for i in ids) and end is not None, "sentinel tokens missing from the tokenizer"
    method = args.cm3_mode
    tokens = ids[:lam] if method == "fixed" else ids
    return CausalMaskedDocumentToSequenceDataset(
        sentinel_token_expectation=lam, sentinel_tokens=tokens, sentinel_method=method, sentinel_eos=end,
        allow_rotation_across_eod=bool(args.cm3_allow_across_eod_boundaries), eod=task.eod, dataset=d2s.dataset,
        block_size=d2s.block_size, break_mode=d2s.break_mode, drop_last=d2s.drop_last, padding_idx=d2s.padding_idx,
        shuffle_buffer_size=d2s.shuffle_buffer_size, seed=d2s.document_shuffle_seed, len_cache=d2s.len_cache, to_skip=d2s.to_skip,
        permute_documents=d2s.permute_documents, source_target=d2s.source_target)
