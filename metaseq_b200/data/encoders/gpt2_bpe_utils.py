"""Byte-level BPE (the GPT-2 scheme) in plain Python, for installations without the ``tokenizers`` package and as
an independent check of it (reference: metaseq/data/encoders/gpt2_bpe_utils.py).

Text is split into word-like chunks by a regular expression; every chunk is turned into bytes, every byte into a
printable stand-in character, and adjacent symbols are merged in the order of the learned merge list until no
listed pair is left.  Symbols are then looked up in the vocabulary.  Decoding reverses the three steps."""
from __future__ import annotations

import json
from functools import lru_cache
from typing import Dict, Iterable, List, Sequence, Set, Tuple

# contractions, letter runs, digit runs, other symbol runs, trailing spaces, spaces before a word
_SPLIT_PATTERN = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""


@lru_cache()
def bytes_to_unicode() -> Dict[int, str]:
    """Byte value -> printable character.  Bytes that already print (``!``..``~``, ``¡``..``¬``, ``®``..``ÿ``) stand
    for themselves; the other 68 are mapped, in ascending order, to the code points from 256 upwards, so that no
    byte becomes whitespace or a control character inside a vocabulary file."""
    printable = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + \
        list(range(ord("®"), ord("ÿ") + 1))
    keep = set(printable)
    table = {b: chr(b) for b in printable}
    spare = 256
    for b in range(256):
        if b not in keep:
            table[b] = chr(spare)
            spare += 1
    return table


def get_pairs(word: Sequence[str]) -> Set[Tuple[str, str]]:
    """The set of adjacent symbol pairs of ``word``."""
    return set(zip(word[:-1], word[1:]))


class Encoder:
    def __init__(self, encoder: Dict[str, int], bpe_merges: Iterable[Tuple[str, str]], errors: str = "replace"):
        import regex

        self.encoder = encoder
        self.decoder = {i: s for s, i in encoder.items()}
        self.errors = errors  # how undecodable byte sequences are handled in decode
        self.byte_encoder = bytes_to_unicode()
        self.byte_decoder = {c: b for b, c in self.byte_encoder.items()}
        self.bpe_ranks = {tuple(pair): rank for rank, pair in enumerate(bpe_merges)}
        self.cache: Dict[str, str] = {}
        self.pat = regex.compile(_SPLIT_PATTERN)

    def bpe(self, token: str) -> str:
        """``token`` (already in stand-in characters) as space-separated merged symbols."""
        hit = self.cache.get(token)
        if hit is not None:
            return hit
        symbols: List[str] = list(token)
        while len(symbols) > 1:
            # the pair that was learned first wins; it is merged at every position where it occurs
            ranked = [(self.bpe_ranks.get(p, None), p) for p in get_pairs(symbols)]
            ranked = [rp for rp in ranked if rp[0] is not None]
            if not ranked:
                break
            _, (left, right) = min(ranked)
            merged: List[str] = []
            i = 0
            while i < len(symbols):
                if i + 1 < len(symbols) and symbols[i] == left and symbols[i + 1] == right:
                    merged.append(left + right)
                    i += 2
                else:
                    merged.append(symbols[i])
                    i += 1
            symbols = merged
        out = " ".join(symbols)
        self.cache[token] = out
        return out

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        for chunk in self.pat.findall(text):
            stand_in = "".join(self.byte_encoder[b] for b in chunk.encode("utf-8"))
            ids.extend(self.encoder[s] for s in self.bpe(stand_in).split(" "))
        return ids

    def decode(self, tokens: Iterable[int]) -> str:
        stand_in = "".join(self.decoder.get(int(t), "") for t in tokens)
        raw = bytearray(self.byte_decoder[c] for c in stand_in)
        return raw.decode("utf-8", errors=self.errors)


def get_encoder(encoder_json_path: str, vocab_bpe_path: str) -> Encoder:
    """Builds the encoder from ``encoder.json`` (symbol -> id) and ``vocab.bpe`` (a version line, then one merge per
    line)."""
    with open(encoder_json_path, "r", encoding="utf-8") as f:
        vocab = json.load(f)
    with open(vocab_bpe_path, "r", encoding="utf-8") as f:
        lines = f.read().split("\n")
    if lines and lines[0].startswith("#"):
        lines = lines[1:]
    merges = [tuple(ln.split()) for ln in lines if len(ln.split()) == 2]
    return Encoder(encoder=vocab, bpe_merges=merges)
