"""BPE / tokenizer registries (``--bpe``, ``--tokenizer``): ``hf_byte_bpe`` wraps HuggingFace
``tokenizers`` byte-level BPE, ``gpt2`` is the same algorithm configured from the GPT-2
``encoder.json`` / ``vocab.bpe`` files (reference: metaseq/data/encoders/)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from metaseq_b200 import registry
from metaseq_b200.dataclass.configs import MetaseqDataclass, opt

build_tokenizer, register_tokenizer, TOKENIZER_REGISTRY, _ = registry.setup_registry("--tokenizer", default=None)
build_bpe, register_bpe, BPE_REGISTRY, _ = registry.setup_registry("--bpe", default=None)


@dataclass
class HuggingFaceByteLevelBPEConfig(MetaseqDataclass):
    bpe_merges: Optional[str] = opt(None, "path to merges.txt")
    bpe_vocab: Optional[str] = opt(None, "path to vocab.json")
    bpe_add_prefix_space: bool = opt(False, "add prefix space before encoding")
    hf_tokenizer: Optional[str] = opt(None, "path to a unified tokenizer file; takes precedence over vocab + merges")


@register_bpe("hf_byte_bpe", dataclass=HuggingFaceByteLevelBPEConfig)
class HuggingFaceByteLevelBPE:
    def __init__(self, cfg):
        try:
            from tokenizers import ByteLevelBPETokenizer, Tokenizer
        except ImportError:
            raise ImportError("Please install huggingface/tokenizers with: pip install tokenizers")
        from metaseq_b200 import file_utils

        if getattr(cfg, "hf_tokenizer", None):
            self.bpe = Tokenizer.from_file(cfg.hf_tokenizer)
        else:
            # either may be a URL: fetched into the local cache once
            self.bpe = ByteLevelBPETokenizer(file_utils.cached_path(cfg.bpe_vocab), file_utils.cached_path(cfg.bpe_merges),
                                             add_prefix_space=cfg.bpe_add_prefix_space)

    def encode(self, x: str) -> str:
        return " ".join(map(str, self.bpe.encode(x).ids))

    def decode(self, x: str) -> str:
        return self.bpe.decode([int(tok) if tok not in {"<unk>", "<mask>"} else tok for tok in x.split()])

    def is_beginning_of_word(self, x: str) -> bool:
        return self.decode(x).startswith(" ")


@dataclass
class GPT2BPEConfig(MetaseqDataclass):
    gpt2_encoder_json: Optional[str] = opt(None, "path to encoder.json")
    gpt2_vocab_bpe: Optional[str] = opt(None, "path to vocab.bpe")


@register_bpe("gpt2", dataclass=GPT2BPEConfig)
class GPT2BPE:
    def __init__(self, cfg):
        try:
            from tokenizers import ByteLevelBPETokenizer

            self.bpe = ByteLevelBPETokenizer(cfg.gpt2_encoder_json, cfg.gpt2_vocab_bpe)
            self._ids = lambda text: self.bpe.encode(text).ids
        except ImportError:  # the plain-Python implementation of the same scheme
            from .gpt2_bpe_utils import get_encoder

            self.bpe = get_encoder(cfg.gpt2_encoder_json, cfg.gpt2_vocab_bpe)
            self._ids = self.bpe.encode

    def encode(self, x: str) -> str:
        return " ".join(map(str, self._ids(x)))

    def decode(self, x: str) -> str:
        return self.bpe.decode([int(tok) for tok in x.split() if tok.isdigit()])

    def is_beginning_of_word(self, x: str) -> bool:
        return self.decode(x).startswith(" ")
