"""Decoding rules of ``SequenceGenerator`` against a model whose next-token distribution is written by hand:
stop tokens, ``min_len``, returned distributions, repetition penalties, the factual-nucleus decay of p, and the
ordering of several samples per prompt."""
import math

import pytest
import torch

from metaseq_b200.data import Dictionary
from metaseq_b200.sequence_generator import SequenceGenerator


class TableDecoder(torch.nn.Module):
    """``logits[next] = table[last token]``: one row of hand-written logits per current token."""

    def __init__(self, table):
        super().__init__()
        self.table = table

    def forward(self, tokens, incremental_state=None, **kw):
        return self.table[tokens], None


class TableModel(torch.nn.Module):
    def __init__(self, table):
        super().__init__()
        self.decoder = TableDecoder(table)

    def forward(self, tokens, **kw):
        return self.decoder(tokens, **kw)

    def max_decoder_positions(self):
        return 24


def _dictionary(n=8):
    d = Dictionary()
    for i in range(n):
        d.add_symbol(f"w{i}")
    return d


def _chain_table(d, successor, strength=8.0):
    """Token t is followed by ``successor[t]`` with overwhelming probability."""
    V = len(d)
    table = torch.full((V, V), -strength)
    for t in range(V):
        table[t, successor.get(t, d.eos())] = strength
    return table


def test_stop_token_ends_a_sample_and_min_len_postpones_it():
    d = _dictionary()
    a, b, c, e = d.index("w0"), d.index("w1"), d.index("w2"), d.index("w3")
    table = _chain_table(d, {d.eos(): a, a: b, b: c, c: e, e: a})
    src = torch.tensor([[d.eos(), a]])
    plain = SequenceGenerator(TableModel(table), d, beam_size=1, max_len_b=10, topp=-1.0)
    toks = plain._generate({"net_input": {"src_tokens": src}})["tokens"][0, 0].tolist()
    assert toks[:6] == [d.eos(), a, b, c, e, a]
    stopping = SequenceGenerator(TableModel(table), d, beam_size=1, max_len_b=10, topp=-1.0, stop=[c])
    toks = stopping._generate({"net_input": {"src_tokens": src}})["tokens"][0, 0].tolist()
    assert toks[:4] == [d.eos(), a, b, c] and set(toks[4:]) <= {d.eos(), d.pad()}
    # with min_len the stop token (and EOS) are banned until that length: the second-best continuation is taken
    table2 = table.clone()
    table2[b, e] = 4.0  # after b: c is best, e second
    late = SequenceGenerator(TableModel(table2), d, beam_size=1, max_len_b=10, min_len=6, topp=-1.0, stop=[c])
    toks = late._generate({"net_input": {"src_tokens": src}})["tokens"][0, 0].tolist()
    assert toks[:4] == [d.eos(), a, b, e] and c not in toks[:6]


def test_returned_distributions_are_the_log_softmax_of_the_model():
    d = _dictionary()
    torch.manual_seed(0)
    table = torch.randn(len(d), len(d))
    src = torch.tensor([[d.eos(), d.index("w0"), d.index("w4")]])
    gen = SequenceGenerator(TableModel(table), d, beam_size=1, max_len_b=8, topp=-1.0, need_logprobs=True)
    out = gen._generate({"net_input": {"src_tokens": src}})
    toks, scores, dist = out["tokens"][0, 0], out["scores"][0, 0], out["distributions"][0, 0]
    # prompt positions: the distribution over position i is the model's prediction after token i-1
    for i in (1, 2):
        want = torch.log_softmax(table[toks[i - 1]], -1)
        assert torch.allclose(dist[i], want, atol=1e-5)
        assert scores[i].item() == pytest.approx(want[toks[i]].item(), abs=1e-5)
    # generated positions: the chosen token is the arg-max of the returned (ban-adjusted) distribution
    for i in range(3, 7):
        if toks[i] in (d.eos(), d.pad()):
            break
        assert int(dist[i].argmax()) == int(toks[i])
        assert scores[i].item() == pytest.approx(dist[i][toks[i]].item(), abs=1e-5)


def test_presence_and_frequency_penalties_break_a_loop():
    d = _dictionary()
    a, b = d.index("w0"), d.index("w1")
    table = torch.full((len(d), len(d)), -6.0)
    table[:, a] = 2.0  # every context prefers a ...
    table[:, b] = 1.0  # ... and b second
    src = torch.tensor([[d.eos(), d.index("w5")]])
    loop = SequenceGenerator(TableModel(table), d, beam_size=1, max_len_b=8, min_len=8, topp=-1.0)
    toks = loop._generate({"net_input": {"src_tokens": src}})["tokens"][0, 0].tolist()
    assert toks[2:7] == [a] * 5
    # gap between a and b in log-probability is 1: a presence penalty above it flips the choice once a was used
    pres = SequenceGenerator(TableModel(table), d, beam_size=1, max_len_b=8, min_len=8, topp=-1.0, alpha_presence=1.5)
    toks = pres._generate({"net_input": {"src_tokens": src}})["tokens"][0, 0].tolist()
    assert toks[2] == a and toks[3] == b
    # a frequency penalty of 0.6 per use needs two uses of a before b overtakes it
    freq = SequenceGenerator(TableModel(table), d, beam_size=1, max_len_b=8, min_len=8, topp=-1.0, alpha_frequency=0.6)
    toks = freq._generate({"net_input": {"src_tokens": src}})["tokens"][0, 0].tolist()
    assert toks[2:4] == [a, a] and toks[4] == b
    # penalties on tokens of the prompt
    src2 = torch.tensor([[d.eos(), a]])
    srcp = SequenceGenerator(TableModel(table), d, beam_size=1, max_len_b=6, min_len=6, topp=-1.0, alpha_presence_src=1.5)
    toks = srcp._generate({"net_input": {"src_tokens": src2}})["tokens"][0, 0].tolist()
    assert toks[2] == b


def test_factual_nucleus_decays_p_and_resets_after_a_full_stop():
    d = Dictionary()
    for sym in ("alpha", "beta", "end.", "gamma"):
        d.add_symbol(sym)
    gen = SequenceGenerator(TableModel(torch.zeros(len(d), len(d))), d, beam_size=1, max_len_b=8, topp=0.9,
                            lambda_decay=0.5, omega_bound=0.3)
    p = torch.full((3,), 0.9)
    p = gen._decay_topp(p, torch.tensor([d.index("alpha"), d.index("beta"), d.index("end.")]))
    assert p.tolist() == pytest.approx([0.45, 0.45, 0.9])
    p = gen._decay_topp(p, torch.tensor([d.index("alpha"), d.index("alpha"), d.index("alpha")]))
    assert p.tolist() == pytest.approx([0.3, 0.3, 0.45])  # never below omega_bound


def test_samples_of_one_prompt_come_back_best_first():
    d = _dictionary()
    torch.manual_seed(3)
    table = torch.randn(len(d), len(d)) * 2
    src = torch.tensor([[d.eos(), d.index("w2")], [d.eos(), d.index("w6")]])
    gen = SequenceGenerator(TableModel(table), d, beam_size=4, max_len_b=7, min_len=7, temperature=1.0, topp=0.95)
    out = gen._generate({"net_input": {"src_tokens": src}})
    assert out["tokens"].shape[:2] == (2, 4)
    totals = out["scores"].sum(-1)
    assert torch.all(totals[:, :-1] >= totals[:, 1:] - 1e-6)
    for row in range(2):
        assert out["tokens"][row, :, :2].tolist() == [src[row].tolist()] * 4  # every sample keeps its prompt
    assert all(math.isfinite(v) for v in totals.flatten().tolist())


def test_ensemble_averages_probabilities_and_keeps_one_state_per_model():
    from metaseq_b200.sequence_generator import EnsembleModel

    torch.manual_seed(0)
    V = 9
    tables = [torch.randn(V, V) for _ in range(3)]
    tokens = torch.tensor([[2, 4, 5], [2, 7, 1]])
    ens = EnsembleModel([TableModel(t) for t in tables])
    assert ens.has_incremental_states() and not ens.has_encoder() and ens.max_decoder_positions() == 24
    states = ens.new_incremental_states()
    assert len(states) == 3 and all(s is not t for s, t in zip(states, states[1:]))
    lprobs, attn = ens.forward_decoder(tokens, states, temperature=0.5)
    probs = torch.stack([torch.softmax(t[tokens[:, -1]] / 0.5, dim=-1) for t in tables]).mean(0)
    assert attn is None and torch.allclose(lprobs.exp(), probs, atol=1e-6)
    assert torch.allclose(lprobs.exp().sum(-1), torch.ones(2), atol=1e-6)
    single, _ = EnsembleModel([TableModel(tables[0])]).forward_decoder(tokens)
    assert torch.allclose(single, torch.log_softmax(tables[0][tokens[:, -1]], dim=-1), atol=1e-6)
