"""``GeneratorInterface``: load a (possibly tensor-parallel / sharded) checkpoint for inference
and serve OpenAI-style completion requests.

Public behaviour follows the reference (metaseq/hub_utils.py:85-466): ``load_model`` builds the
model for this rank's ``model_part``, switches it to the cached inference path and loads the
weights; ``generate`` takes pre-tokenised prompts plus ``min_tokens / max_tokens /
temperature / top_p / logprobs / n / best_of / echo / stop / seed`` and repetition-penalty
knobs and returns, per prompt, ``n`` dicts with ``text``, ``tokens``, ``text_offset``,
``token_scores`` and ``top_logprobs``; special tokens after the first position end a result.
"""
from __future__ import annotations

import ast
import logging
import os
import time
from argparse import Namespace
from typing import Any, Dict, List, Optional

import torch

from metaseq_b200 import checkpoint_utils, tasks, utils
from metaseq_b200.dataclass.utils import Cfg
from metaseq_b200.parallel import utils as dist_utils
from metaseq_b200.parallel.fsdp import fsdp_enable_wrap, fsdp_wrap
from metaseq_b200.trainer import utils_resolve_max_positions

logger = logging.getLogger(__name__)


class _IdTextCodec:
    """Fallback codec when no BPE files are configured: tokens are rendered as ``<id>``."""

    class _Enc:
        def __init__(self, offsets):
            self.offsets = offsets

    def decode(self, ids):
        return "".join(f"<{int(i)}>" for i in ids)

    def encode(self, text):
        offs, pos = [], 0
        for part in text.split(">"):
            if part:
                offs.append((pos, pos + len(part) + 1))
                pos += len(part) + 1
        return self._Enc(offs)


def tensorize_input(tokenizer, prompt: str) -> torch.Tensor:
    """``[1, T + 1]`` token ids of ``prompt`` with token 0 in front (metaseq/hub_utils.py:32)."""
    ids = tokenizer.encode(prompt).ids
    return torch.tensor([[0] + list(ids)], dtype=torch.long)


def get_next_token(logits: torch.Tensor, tokenizer) -> str:
    """Text of the most probable next token after the last position of the first sequence, without the
    byte-level BPE's space marker (metaseq/hub_utils.py:39)."""
    best = int(torch.argmax(logits[0, -1], dim=-1))
    return tokenizer.decode([best]).replace("\u0120", "")


def setup_vocab_and_merges(model_path: str):
    """Paths of the GPT-2 vocabulary and merges files kept beside a model, and the tokenizer built from them
    (metaseq/hub_utils.py:46)."""
    from tokenizers import ByteLevelBPETokenizer

    vocab_file = os.path.join(model_path, "gpt2-vocab.json")
    merges_file = os.path.join(model_path, "gpt2-merges.txt")
    return vocab_file, merges_file, ByteLevelBPETokenizer.from_file(vocab_file, merges_file)


class _EncoderHubInterface:
    """``encode`` / ``decode`` of one registered text encoder, built from keyword arguments."""

    _kind = ""

    def __init__(self, name, **kwargs):
        from metaseq_b200.data import encoders

        build = encoders.build_bpe if self._kind == "bpe" else encoders.build_tokenizer
        self._impl = build(Namespace(**{self._kind: name}, **kwargs))
        assert self._impl is not None, f"unknown {self._kind}: {name}"
        setattr(self, self._kind, self._impl)

    def encode(self, sentence: str) -> str:
        return self._impl.encode(sentence)

    def decode(self, sentence: str) -> str:
        return self._impl.decode(sentence)


class BPEHubInterface(_EncoderHubInterface):
    """Byte-pair encoder by registry name (metaseq/hub_utils.py:53-66)."""

    _kind = "bpe"


class TokenizerHubInterface(_EncoderHubInterface):
    """Word tokenizer by registry name (metaseq/hub_utils.py:69-82)."""

    _kind = "tokenizer"


class GeneratorInterface:
    def __init__(self, cfg):
        self.cfg = cfg
        if isinstance(self.cfg, Namespace):
            from metaseq_b200.dataclass.utils import convert_namespace_to_config

            self.cfg = convert_namespace_to_config(self.cfg)
        self.models = None
        self.task = None
        self.bpe = None

    # ---------------------------------------------------------------- loading
    def load_model(self):
        cfg = self.cfg
        utils_import = getattr(cfg.common, "user_dir", None)
        if utils_import:
            from metaseq_b200 import options

            options._import_user_module(cfg.common)
        if cfg.dataset.max_tokens is None and cfg.dataset.batch_size is None:
            cfg.dataset.batch_size = 1
        logger.info(f"loading model(s) from {cfg.common_eval.path}")
        r = dist_utils.get_global_rank()
        # which shard files exist decides between consolidated and sharded loading
        path = cfg.common_eval.path
        suffix = cfg.checkpoint.checkpoint_suffix
        sharded_candidates = [f"{path[:-3]}{suffix}-shard0.pt" if path.endswith(".pt") else path]
        if cfg.distributed_training.use_sharded_state or any(os.path.exists(p) for p in sharded_candidates):
            if any(os.path.exists(p) for p in sharded_candidates):
                suffix += f"-shard{dist_utils.get_data_parallel_rank()}"
        task = tasks.setup_task(cfg.task)

        def _build_model(cfg_, task_):
            cfg_.model.tensor_parallel_init_model_on_gpu = torch.cuda.is_available() and not cfg.common.cpu
            model = task_.build_model(cfg_.model)
            if torch.cuda.is_available() and not cfg.common.cpu:
                model = model.cuda()
            model.make_generation_fast_()
            return fsdp_wrap(model)

        with fsdp_enable_wrap(cfg.distributed_training, use_sharded_state=cfg.distributed_training.use_sharded_state):
            models, _model_cfg, task = checkpoint_utils.load_model_ensemble_and_task(
                cfg.common_eval.path.split(os.pathsep),
                arg_overrides=ast.literal_eval(cfg.common_eval.model_overrides),
                task=task, suffix=suffix, strict=True, num_shards=cfg.checkpoint.checkpoint_shard_count,
                build_model_hook=_build_model)
        self._finish_setup(models, task)
        logger.info(f"loaded model {r}")
        return models

    def _finish_setup(self, models, task):
        cfg = self.cfg
        self.task = task
        self.models = models
        for m in models:
            if cfg.common.fp16 or cfg.common.memory_efficient_fp16:
                m.half()
            elif cfg.common.bf16:
                m.bfloat16()
            if torch.cuda.is_available() and not cfg.common.cpu:
                m.cuda()
            if hasattr(m, "make_generation_fast_"):
                m.make_generation_fast_()
        self.src_dict = task.source_dictionary
        self.tgt_dict = task.target_dictionary
        self.bpe = self._build_bpe(task)
        self.max_positions = utils_resolve_max_positions(task.max_positions(), *[m.max_positions() for m in models])
        self._pad_token_ind = self.tgt_dict.pad_index
        self._special_token_inds = {self.tgt_dict.eos_index, self.tgt_dict.pad_index, self.tgt_dict.bos_index,
                                    self.tgt_dict.unk_index}

    def _build_bpe(self, task):
        class _Holder:
            pass

        holder = _Holder()
        tok = getattr(task, "tokenizer", None)
        if tok is None:
            b = getattr(self.cfg, "bpe", None)
            vocab = getattr(b, "bpe_vocab", None) if b is not None else None
            merges = getattr(b, "bpe_merges", None) if b is not None else None
            unified = getattr(b, "hf_tokenizer", None) if b is not None else None
            if unified and os.path.exists(unified):
                from tokenizers import Tokenizer

                tok = Tokenizer.from_file(unified)
            elif vocab and merges and os.path.exists(vocab) and os.path.exists(merges):
                from tokenizers import ByteLevelBPETokenizer

                tok = ByteLevelBPETokenizer.from_file(vocab, merges)
        holder.bpe = tok if tok is not None else _IdTextCodec()
        return holder

    @classmethod
    def from_model(cls, cfg, model, task):
        """Wraps an already-built model (tests, notebooks)."""
        self = cls(cfg)
        self._finish_setup([model], task)
        return self

    # -------------------------------------------------------------- tokenizer
    def encode_fn(self, x: str):
        """Token ids of ``x``; line ends are normalised to ``\\n`` first (browsers send ``\\r\\n``)."""
        from metaseq_b200.service.utils import normalize_newlines

        assert self.bpe is not None
        return self.bpe.bpe.encode(normalize_newlines(x)).ids

    def decode_fn(self, x: List[int]) -> str:
        assert self.bpe is not None
        return self.bpe.bpe.decode(x)

    # ---------------------------------------------------------------- generate
    def generate(self, inputs: List[List[int]], min_tokens: List[int] = None, max_tokens: List[int] = None,
                 temperature: float = 1.0, top_p: float = -1.0, logprobs: int = 0, n: int = 1,
                 best_of: Optional[int] = None, echo: bool = False, stop: Optional[List[int]] = None,
                 seed: Optional[int] = None, use_cuda: bool = True, omega_bound: float = 0.3,
                 lambda_decay: float = -1, alpha_presence: float = 0.0, alpha_frequency: float = 0.0,
                 alpha_presence_src: float = 0.0, alpha_frequency_src: float = 0.0,
                 alpha_src_penalty_end_idx: int = -1):
        if seed:
            utils.set_torch_seed(seed)
        t_start = time.time()
        gen_time = 0.0
        best_of = best_of or n
        assert best_of >= n
        gen = self.cfg.generation
        gen.sampling_topp = top_p if top_p > 0 else -1
        gen.sampling = top_p > 0.0
        gen.beam = best_of
        if temperature > 0:
            gen.temperature = temperature
        elif temperature == 0:
            gen.sampling, gen.temperature, gen.sampling_topp = False, 1.0, -1
        else:
            raise ValueError("temperature must be >= 0 and <= 1")
        max_seq = self.max_positions
        use_cuda = use_cuda and torch.cuda.is_available() and not self.cfg.common.cpu
        results: List[Any] = [None] * len(inputs)
        tokens = [torch.LongTensor(t) for t in inputs]
        lengths = [len(t) for t in inputs]
        dataset = self.task.build_dataset_for_inference(tokens, lengths)
        batches = self.task.get_batch_iterator(
            dataset=dataset, max_tokens=None, max_sentences=len(inputs), max_positions=None,
            ignore_invalid_inputs=False, skip_remainder_batch=False, batch_by_size=False,
        ).next_epoch_itr(shuffle=False)
        for batch in batches:
            src_tokens = batch["net_input"]["src_tokens"]
            src_lengths = batch["net_input"]["src_lengths"]
            ids = batch["id"].tolist()
            bsz = src_tokens.size(0)
            mx = [max_tokens[i] for i in ids] if max_tokens is not None else [max_seq] * bsz
            mn = [min_tokens[i] for i in ids] if min_tokens is not None else [0] * bsz
            longest = int(src_lengths.max())
            gen.max_len_b = min(max_seq, max(mx) + longest)
            gen.min_len = max(mn) + longest
            gen.max_len_a = 0
            generator = self.task.build_generator(self.models, gen, extra_gen_cls_kwargs={
                "stop": stop, "need_logprobs": logprobs > 0, "omega_bound": omega_bound,
                "lambda_decay": lambda_decay, "alpha_presence": alpha_presence, "alpha_frequency": alpha_frequency,
                "alpha_presence_src": alpha_presence_src, "alpha_frequency_src": alpha_frequency_src,
                "alpha_src_penalty_end_idx": alpha_src_penalty_end_idx})
            if use_cuda:
                batch = utils.move_to_cuda(batch)
            t0 = time.time()
            out = self.task.inference_step(generator, self.models, batch)
            gen_time += time.time() - t0
            all_tokens = out["tokens"].cpu()
            all_scores = out["scores"].cpu()
            all_dist = out["distributions"].cpu() if logprobs > 0 else None
            for row, sample_id in enumerate(ids):
                prompt_len = lengths[sample_id]
                beams = []
                for j in range(n):
                    beams.append(self._format_one(
                        all_tokens[row, j].tolist(), all_scores[row, j].tolist(),
                        all_dist[row, j] if all_dist is not None else None, prompt_len, mx[row], echo, logprobs))
                results[sample_id] = beams
        logger.info("Total time: {:.3f} seconds; generation time: {:.3f}".format(time.time() - t_start, gen_time))
        return results

    def _format_one(self, toks, scores, dist, prompt_len, max_new, echo, logprobs):
        toks, scores, dist = self._filter_special(self._pad_token_ind, self._special_token_inds, toks, scores, dist)
        if not echo:
            toks = toks[prompt_len + 1:][:max_new]
            scores = scores[prompt_len + 1:][:max_new]
            if dist is not None:
                dist = dist[prompt_len + 1:][:max_new]
        text_tokens = toks[1:] if echo else toks  # the leading </s> is not part of the text
        shown_scores = [None] + scores[1:] if echo else scores
        codec = self.bpe.bpe
        text = codec.decode(text_tokens)
        res = {
            "text": text,
            "tokens": [codec.decode([t]) for t in toks],
            "text_offset": [s for s, _ in codec.encode(text).offsets],
            "token_scores": shown_scores,
        }
        if logprobs > 0 and dist is not None:
            top_scores, top_toks = dist.topk(k=logprobs, dim=-1)
            per_pos = [{codec.decode([int(t)]): float(s) for t, s in zip(tt, ss)} for tt, ss in zip(top_toks, top_scores)]
            res["top_logprobs"] = [None] + per_pos[1:] if echo else per_pos
        else:
            res["top_logprobs"] = None
        return res

    @staticmethod
    def _filter_special(pad_token_ind, special_token_inds, tokens: List[int], scores: List[float], distributions):
        """Drops pads and cuts the sequence at the first special token after position 0."""
        kept_t, kept_s, mask = [], [], []
        for i, (t, s) in enumerate(zip(tokens, scores)):
            if t == pad_token_ind:
                mask.append(False)
                continue
            if t in special_token_inds and i > 0:
                mask.append(False)
                break
            mask.append(True)
            kept_t.append(t)
            kept_s.append(s)
        if distributions is not None:
            assert len(mask) <= distributions.shape[0]
            mask.extend([False] * (distributions.shape[0] - len(mask)))
            distributions = distributions[torch.tensor(mask, dtype=torch.bool)]
        return kept_t, kept_s, distributions
