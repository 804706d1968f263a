"""Batched incremental generation: one prefill over the prompt batch, then one decoder step
per generated token using the key/value cache.

Semantics follow the reference (metaseq/sequence_generator.py:142-344): every prompt is
replicated ``beam_size`` times (independent samples, not a beam search); the batch is
prefilled up to the padded prompt length and each sample's first generated token is sampled
from the distribution at its own prompt length; EOS / pad / stop tokens are banned inside the
prompt; ``min_len`` bans EOS and stop tokens, the last position forces EOS; finished samples
keep emitting EOS; the ``beam_size`` samples of a prompt are returned sorted by cumulative
log-probability.  Sampling is greedy when ``temperature == 0`` or ``topp <= 0`` and nucleus
(top-p) otherwise (:399-437), optionally with the factual-nucleus decay of p over a sentence
(:439-470) and presence / frequency penalties over generated and source tokens (:472-534).
"""
from __future__ import annotations

import logging
import math
import sys
from typing import Dict, List, Optional

import torch
import torch.nn as nn
from torch import Tensor

from metaseq_b200.models.decode_step import GraphedDecodeStep
from metaseq_b200.ops import functional as ops_f

logger = logging.getLogger(__name__)


class SequenceGenerator(nn.Module):
    def __init__(self, models, tgt_dict, beam_size: int = 1, max_len_a: int = 0, max_len_b: int = 200,
                 min_len: int = 1, temperature: float = 1.0, need_logprobs: bool = False,
                 stop: Optional[List[int]] = None, topp: float = -1, profile: bool = False,
                 omega_bound: float = 0.3, lambda_decay: float = -1, alpha_presence: float = 0.0,
                 alpha_frequency: float = 0.0, alpha_presence_src: float = 0.0, alpha_frequency_src: float = 0.0,
                 alpha_src_penalty_end_idx: int = -1, eos_check_interval: int = 1, decode_graph: bool = True):
        super().__init__()
        self.decode_graph = decode_graph  # replay the one-token step from a CUDA graph where the model allows it
        self.model = models[0] if isinstance(models, (list, tuple)) else models
        self.tgt_dict = tgt_dict
        self.pad = tgt_dict.pad()
        self.unk = tgt_dict.unk()
        self.eos = tgt_dict.eos()
        self.vocab_size = len(tgt_dict)
        self.beam_size = min(beam_size, self.vocab_size - 1)
        self.max_len_a = max_len_a
        self.max_len_b = max_len_b
        self.min_len = min_len
        self.need_logprobs = need_logprobs
        self.stop = stop if stop is not None else []
        if topp is None:
            topp = 0.0
        self.sampling_topp = max(0.0, topp)
        self.shard_picks = True  # greedy decoding under tensor parallelism picks tokens from the logit shards
        self.temperature = temperature
        assert temperature >= 0, "--temperature must be >=0"
        self.profile = profile
        self.omega_bound = omega_bound
        self.lambda_decay = lambda_decay
        self.alpha_presence = alpha_presence
        self.alpha_frequency = alpha_frequency
        self.alpha_presence_src = alpha_presence_src
        self.alpha_frequency_src = alpha_frequency_src
        self.alpha_src_penalty_end_idx = alpha_src_penalty_end_idx
        self.eos_check_interval = max(1, eos_check_interval)
        self.model.eval()

    def cuda(self):
        self.model.cuda()
        return self

    @torch.no_grad()
    def forward(self, sample, prefix_tokens=None, bos_token=None):
        return self._generate(sample, prefix_tokens, bos_token=bos_token)

    @torch.no_grad()
    def generate(self, models, sample, **kwargs):
        return self._generate(sample, **kwargs)

    # ------------------------------------------------------------------ core
    def _logprobs(self, logits):
        logits = logits.float()
        if self.temperature > 0 and self.temperature != 1.0:
            logits = logits / self.temperature
        return torch.log_softmax(logits, dim=-1)

    def _generate(self, sample, prefix_tokens: Optional[Tensor] = None, bos_token: Optional[int] = None):
        state: Dict = {}
        src_tokens = sample["net_input"]["src_tokens"]
        src_lengths = (src_tokens.ne(self.eos) & src_tokens.ne(self.pad)).long().sum(dim=1)
        bsz, src_len = src_tokens.shape
        K = self.beam_size
        max_len = int(min(self.model.max_decoder_positions(), self.max_len_b or 1e99))
        min_len = min(max_len, self.min_len or 0)
        assert min_len <= max_len, "min_len cannot be larger than max_len, please adjust these!"
        n = bsz * K
        dev = src_tokens.device
        scores = torch.zeros(n, max_len, device=dev, dtype=torch.float)
        tokens = torch.full((n, max_len), self.pad, device=dev, dtype=torch.long)
        vocab = self.vocab_size
        count_tokens = torch.zeros(n, vocab, device=dev, dtype=torch.long) if self._has_penalties() else None
        count_src = self._count_source_tokens(src_tokens, K, vocab) if self._has_src_penalties() else None
        all_lprobs = torch.zeros(n, max_len, vocab, device=dev, dtype=torch.float) if self.need_logprobs else None

        start = src_len
        tokens[:, :start] = src_tokens.repeat_interleave(K, 0)
        graphed = None
        decoder = getattr(self.model, "decoder", None)
        if self.decode_graph and decoder is not None and max_len > start and GraphedDecodeStep.supported(decoder, n):
            graphed = GraphedDecodeStep.for_decoder(decoder, n, max_len)
            state = graphed.new_state()
        # ---------------------------------------------------------- prefill
        logits, _ = self.model(tokens[:, :start], incremental_state=state)
        if graphed is not None:
            graphed.begin(tokens[:, :start])
        lp_all = self._logprobs(logits)  # [n, start, V]
        if all_lprobs is not None:
            all_lprobs[:, 1:start] = lp_all[:, :-1]
        if start > 1:
            scores[:, 1:start] = lp_all[:, :-1].gather(-1, tokens[:, 1:start].unsqueeze(-1)).squeeze(-1)
        # each sample continues from the distribution at its own prompt length; positions after the
        # prompt carry no score
        plen = src_lengths.repeat_interleave(K, 0)  # [n]
        pos = torch.arange(max_len, device=dev)[None, :]
        scores.masked_fill_(pos > plen[:, None], 0.0)
        lprobs = lp_all.gather(1, plen.clamp(max=start - 1)[:, None, None].expand(n, 1, vocab)).squeeze(1).clone()
        del lp_all, logits
        eos_mask = torch.zeros(n, dtype=torch.bool, device=dev)
        neg_inf = -math.inf
        sentence_p = torch.full((n,), self.sampling_topp, device=dev) if self.lambda_decay > 0 else None
        # Greedy decoding over vocabulary-parallel logits picks the token from the shards: the graphed step returns
        # this rank's columns and a record of four numbers per row and rank replaces the gather of [n, V] logits.
        sharded = (graphed is not None and getattr(graphed, "tp", 1) > 1 and self._is_greedy() and count_tokens is None
                   and count_src is None and all_lprobs is None and self.temperature in (0.0, 1.0)
                   and self.shard_picks)
        local = None
        # ------------------------------------------------------- decode loop
        for step in range(start, max_len):
            if sharded and local is not None:
                banned = [self.pad]
                if step < min_len and step < max_len - 1:
                    banned += [self.eos, *self.stop]
                next_scores, next_toks = graphed.pick_greedy(local, banned=banned,
                                                             only=self.eos if step >= max_len - 1 else None)
                # finished hypotheses can only repeat EOS, at no cost
                next_toks = torch.where(eos_mask, torch.full_like(next_toks, self.eos), next_toks)
                next_scores = torch.where(eos_mask, torch.zeros_like(next_scores), next_scores)
                tokens[:, step] = next_toks
                scores[:, step] = next_scores
                eos_mask |= next_toks == self.eos
                for s in self.stop:
                    eos_mask |= next_toks == s
                if (step - start) % self.eos_check_interval == 0 and bool(eos_mask.all()):
                    break
                if step + 1 >= max_len:
                    break
                local = graphed.step(tokens[:, step], gather=False)
                continue
            if step < min_len and step < max_len - 1:  # the forced EOS of the last position wins over min_len
                lprobs[:, self.eos] = neg_inf
                for s in self.stop:
                    lprobs[:, s] = neg_inf
            lprobs = torch.where(torch.isnan(lprobs), torch.full_like(lprobs, neg_inf), lprobs)
            lprobs[:, self.pad] = neg_inf
            if step >= max_len - 1:
                lprobs[:, : self.eos] = neg_inf
                lprobs[:, self.eos + 1:] = neg_inf
            if count_tokens is not None or count_src is not None:
                lprobs = self._apply_repetition_penalties(lprobs, count_tokens, count_src)
            # finished hypotheses can only repeat EOS
            keep = lprobs[:, self.eos].clone()
            lprobs[eos_mask] = neg_inf
            lprobs[:, self.eos] = torch.where(eos_mask, torch.zeros_like(keep), keep)
            next_scores, next_toks = self._sample(lprobs, sentence_p)
            if sentence_p is not None:
                sentence_p = self._decay_topp(sentence_p, next_toks)
            if count_tokens is not None:
                count_tokens.scatter_add_(1, next_toks[:, None], torch.ones_like(next_toks[:, None]))
            tokens[:, step] = next_toks
            scores[:, step] = next_scores
            if all_lprobs is not None:
                all_lprobs[:, step] = lprobs
            eos_mask |= next_toks == self.eos
            for s in self.stop:
                eos_mask |= next_toks == s
            if (step - start) % self.eos_check_interval == 0 and bool(eos_mask.all()):
                break
            if step + 1 >= max_len:
                break
            if sharded:
                local = graphed.step(tokens[:, step], gather=False)  # from here on the tokens come from the shards
            elif graphed is not None:
                lprobs = self._logprobs(graphed.step(tokens[:, step]))
            else:
                logits, _ = self.model.decoder(tokens[:, : step + 1], incremental_state=state)
                lprobs = self._logprobs(logits[:, -1, :])
        # ------------------------------------------------- order the samples
        total = scores.view(bsz, K, -1).sum(dim=-1)
        order = total.sort(dim=-1, descending=True).indices
        flat = (order + K * torch.arange(bsz, device=dev).unsqueeze(1)).view(-1)
        out = {"tokens": tokens[flat].view(bsz, K, -1), "scores": scores[flat].view(bsz, K, -1)}
        if all_lprobs is not None:
            out["distributions"] = all_lprobs[flat].view(bsz, K, -1, vocab)
        return out

    # -------------------------------------------------------------- sampling
    def _is_greedy(self) -> bool:
        return self.temperature == 0.0 or self.sampling_topp == 0.0

    def _sample(self, lprobs: Tensor, sentence_p: Optional[Tensor] = None):
        """Returns ``(log-prob of the chosen token, chosen token)`` per row."""
        if self.temperature == 0.0 or self.sampling_topp == 0.0:
            best = lprobs.max(dim=-1)
            return best.values, best.indices
        if lprobs.is_cuda and lprobs.dtype == torch.float32 and lprobs.shape[-1] <= 56000 and ops_f.get_backend() != "torch":
            # one kernel per step instead of sort + cumsum + mask + renormalise + multinomial over [rows, V]
            p = sentence_p if sentence_p is not None else self.sampling_topp
            return ops_f.sample_top_p(lprobs, p)
        probs = torch.exp(lprobs)
        sprobs, sidx = probs.sort(descending=True, dim=-1)
        csum = sprobs.cumsum(dim=-1)
        p = sentence_p[:, None] if sentence_p is not None else self.sampling_topp
        # keep the smallest prefix whose mass reaches p (always at least the top token)
        cut = (csum - sprobs) >= p
        sprobs = torch.nan_to_num(sprobs.masked_fill(cut, 0.0), nan=0.0, posinf=0.0)
        mass = sprobs.sum(dim=-1, keepdim=True)
        # a row without any admissible token (everything banned) takes the first sorted entry instead of
        # handing multinomial an all-zero row
        sprobs[:, :1] = torch.where(mass > 0, sprobs[:, :1], torch.ones_like(mass))
        sprobs = sprobs / sprobs.sum(dim=-1, keepdim=True)
        choice = torch.multinomial(sprobs, 1)
        toks = sidx.gather(-1, choice).squeeze(-1)
        chosen = lprobs.gather(-1, toks[:, None]).squeeze(-1)
        return chosen, toks

    def _sample_topp(self, lprobs):
        return self._sample(lprobs)

    def _decay_topp(self, sentence_p: Tensor, next_toks: Tensor) -> Tensor:
        """Factual nucleus: p decays by ``lambda_decay`` per token down to ``omega_bound`` and is
        reset at the end of a sentence (a token whose text ends with a full stop)."""
        sentence_p = torch.clamp(sentence_p * self.lambda_decay, min=self.omega_bound)
        period_ids = getattr(self, "_period_ids", None)
        if period_ids is None:
            ids = [i for i in range(min(len(self.tgt_dict), self.vocab_size)) if str(self.tgt_dict[i]).endswith(".")]
            period_ids = torch.tensor(ids or [self.eos], device=next_toks.device)
            self._period_ids = period_ids
        reset = torch.isin(next_toks, period_ids)
        return torch.where(reset, torch.full_like(sentence_p, self.sampling_topp), sentence_p)

    # ------------------------------------------------------------- penalties
    def _has_penalties(self) -> bool:
        return self.alpha_presence > 0 or self.alpha_frequency > 0

    def _has_src_penalties(self) -> bool:
        return self.alpha_presence_src > 0 or self.alpha_frequency_src > 0

    def _count_source_tokens(self, src_tokens, K, vocab):
        src = src_tokens.repeat_interleave(K, 0)
        if self.alpha_src_penalty_end_idx > 0:
            src = src[:, : self.alpha_src_penalty_end_idx]
        counts = torch.zeros(src.shape[0], vocab, device=src.device, dtype=torch.long)
        counts.scatter_add_(1, src, torch.ones_like(src))
        counts[:, self.pad] = 0
        return counts

    def _apply_repetition_penalties(self, lprobs, count_tokens, count_src):
        """OpenAI-style penalties on the (log-)scores: ``alpha_frequency * count`` plus
        ``alpha_presence`` for every token already present."""
        if count_tokens is not None:
            lprobs = lprobs - self.alpha_frequency * count_tokens - self.alpha_presence * (count_tokens > 0)
        if count_src is not None:
            lprobs = lprobs - self.alpha_frequency_src * count_src - self.alpha_presence_src * (count_src > 0)
        return lprobs

    def _update_repetition_counts(self, next_toks, count_tokens):
        if count_tokens is not None:
            count_tokens.scatter_add_(1, next_toks[:, None], torch.ones_like(next_toks[:, None]))
        return count_tokens


class EnsembleModel(nn.Module):
    """Several decoder-only language models scored as one: each model keeps its own incremental state and the
    next-token distribution is the arithmetic mean of the models' probabilities (log-sum-exp of their log-probs
    minus log n).  With one model it is that model's log-softmax.  Reference: metaseq/sequence_generator.py:537-685;
    the encoder-side and alignment variants there (``forward_encoder``, ``SequenceGeneratorWithAlignment``) belong
    to encoder-decoder models, which neither code base defines."""

    def __init__(self, models):
        super().__init__()
        models = list(models)
        assert len(models) > 0
        self.models_size = len(models)
        self.single_model = models[0]
        self.models = nn.ModuleList(models)
        self.has_incremental = all(hasattr(m, "decoder") for m in models)

    def forward(self):  # scoring goes through forward_decoder
        raise RuntimeError("call forward_decoder")

    def set_decoder_beam_size(self, beam_size):
        """Tells models that specialise on the beam width (``set_beam_size``) what it is."""
        if beam_size > 1:
            for model in self.models:
                if hasattr(model, "set_beam_size"):
                    model.set_beam_size(beam_size)

    def forward_encoder(self, net_input):
        """Decoder-only models have no encoder pass: always ``None``."""
        return None

    def reorder_encoder_out(self, encoder_outs, new_order):
        """Nothing to reorder without an encoder: an empty list."""
        return []

    def has_encoder(self) -> bool:
        return hasattr(self.single_model, "encoder")

    def has_incremental_states(self) -> bool:
        return self.has_incremental

    def max_decoder_positions(self) -> int:
        limits = [m.max_decoder_positions() for m in self.models if hasattr(m, "max_decoder_positions")]
        return min([x for x in limits if x is not None] + [sys.maxsize])

    def new_incremental_states(self):
        return [{} for _ in range(self.models_size)]

    @torch.no_grad()
    def forward_decoder(self, tokens: Tensor, incremental_states=None, temperature: float = 1.0):
        """``tokens``: [B, T] prefix.  Returns ([B, V] log-probabilities of the next token, None)."""
        per_model = []
        for i, model in enumerate(self.models):
            if self.has_incremental and incremental_states is not None:
                out = model.decoder(tokens, incremental_state=incremental_states[i])
            elif hasattr(model, "decoder"):
                out = model.decoder(tokens)
            else:
                out = model(tokens)
            logits = out[0] if isinstance(out, (tuple, list)) else out
            last = logits[:, -1, :].float()
            if temperature != 1.0:
                last = last / temperature
            per_model.append(torch.log_softmax(last, dim=-1))
        if self.models_size == 1:
            return per_model[0], None
        return torch.logsumexp(torch.stack(per_model, dim=0), dim=0) - math.log(self.models_size), None

    def reorder_incremental_state(self, incremental_states, new_order):
        if not self.has_incremental or incremental_states is None:
            return
        for model, state in zip(self.models, incremental_states):
            if hasattr(model.decoder, "reorder_incremental_state"):
                model.decoder.reorder_incremental_state(state, new_order)
