"""Symbol <-> index mapping.

Special symbols occupy indices 0..3 in the order ``<s>, <pad>, </s>, <unk>`` and the
table can be padded with ``madeupwordNNNN`` entries to a multiple (OPT pads the
50265-entry GPT-2 BPE table to 50272 = 8 * 6284).  Reference:
metaseq/data/dictionary.py (specials :22-41, ``pad_to_multiple_`` :189-196).
"""
from __future__ import annotations

import os
from collections import Counter
from typing import Iterable, List, Optional

import torch


class Dictionary:
    def __init__(self, *, bos="<s>", pad="<pad>", eos="</s>", unk="<unk>", extra_special_symbols=None):
        self.bos_word, self.unk_word, self.pad_word, self.eos_word = bos, unk, pad, eos
        self.symbols: List[str] = []
        self.count: List[int] = []
        self.indices = {}
        self.bos_index = self.add_symbol(bos)
        self.pad_index = self.add_symbol(pad)
        self.eos_index = self.add_symbol(eos)
        self.unk_index = self.add_symbol(unk)
        for s in extra_special_symbols or []:
            self.add_symbol(s)
        self.nspecial = len(self.symbols)

    def __eq__(self, other):
        return isinstance(other, Dictionary) and self.indices == other.indices

    def __getitem__(self, idx: int) -> str:
        return self.symbols[idx] if idx < len(self.symbols) else self.unk_word

    def __len__(self) -> int:
        return len(self.symbols)

    def __contains__(self, sym) -> bool:
        return sym in self.indices

    def index(self, sym: str) -> int:
        return self.indices.get(sym, self.unk_index)

    def get_count(self, idx: int) -> int:
        return self.count[idx]

    def string(self, tensor, bpe_symbol=None, escape_unk=False, extra_symbols_to_ignore=None, unk_string=None,
               include_eos=False) -> str:
        """Text of a token tensor (one line per row for a matrix).  End-of-sentence (unless ``include_eos``),
        begin-of-sentence and the given extra symbols are left out; ``bpe_symbol`` (a continuation marker such as
        ``@@ ``) is removed."""
        if torch.is_tensor(tensor) and tensor.dim() == 2:
            rows = (self.string(row, bpe_symbol, escape_unk, extra_symbols_to_ignore, unk_string, include_eos)
                    for row in tensor)
            return "\n".join(rows)
        skipped = {self.bos_index, *(extra_symbols_to_ignore or ())}
        if not include_eos:
            skipped.add(self.eos_index)
        unknown = unk_string if unk_string is not None else self.unk_string(escape_unk)
        words = [unknown if i == self.unk_index else self[i] for i in map(int, tensor) if i not in skipped]
        text = " ".join(words)
        return (text + " ").replace(bpe_symbol, "").rstrip() if bpe_symbol else text

    def unk_string(self, escape=False) -> str:
        return "<{}>".format(self.unk_word) if escape else self.unk_word

    def add_symbol(self, word: str, n: int = 1, overwrite: bool = False) -> int:
        if word in self.indices and not overwrite:
            idx = self.indices[word]
            self.count[idx] += n
            return idx
        idx = len(self.symbols)
        self.indices[word] = idx
        self.symbols.append(word)
        self.count.append(n)
        return idx

    def update(self, new_dict: "Dictionary"):
        """Adds every symbol of ``new_dict`` with its count."""
        for word, c in zip(new_dict.symbols, new_dict.count):
            self.add_symbol(word, c)

    def finalize(self, threshold: int = -1, nwords: int = -1, padding_factor: int = 8):
        """Orders the non-special symbols by falling count (ties alphabetically), keeps at most ``nwords`` entries
        in total and only symbols seen at least ``threshold`` times, then pads to a multiple of ``padding_factor``."""
        keep = self.nspecial
        limit = (nwords if nwords > 0 else len(self)) - keep
        ranked = sorted(zip(self.symbols[keep:], self.count[keep:]), key=lambda sc: (-sc[1], sc[0]))
        ranked = [(sym, n) for sym, n in ranked[:max(limit, 0)] if n >= threshold]
        self.symbols = self.symbols[:keep] + [sym for sym, _ in ranked]
        self.count = self.count[:keep] + [n for _, n in ranked]
        self.indices = {sym: i for i, sym in enumerate(self.symbols)}
        self.pad_to_multiple_(padding_factor)

    def pad_to_multiple_(self, padding_factor: int):
        """Appends ``madeupwordNNNN`` entries (count 0) until the size is a multiple of ``padding_factor``."""
        missing = -len(self) % padding_factor if padding_factor > 1 else 0
        for i in range(missing):
            self.add_symbol(f"madeupword{i:04d}", n=0)

    def bos(self) -> int:
        return self.bos_index

    def pad(self) -> int:
        return self.pad_index

    def eos(self) -> int:
        return self.eos_index

    def unk(self) -> int:
        return self.unk_index

    @classmethod
    def load(cls, f) -> "Dictionary":
        """``<symbol> <count> [#fairseq:overwrite]`` per line."""
        d = cls()
        d.add_from_file(f)
        return d

    def add_from_file(self, f):
        """Appends the entries of a dictionary file (a path or an open text file).  A line that ends in
        ``#fairseq:overwrite`` may redefine a symbol that exists; any other duplicate is an error."""
        if isinstance(f, str):
            with open(f, "r", encoding="utf-8") as handle:
                return self.add_from_file(handle)
        flag = "#fairseq:overwrite"
        for raw in f:
            fields = raw.rstrip().rsplit(" ", 2)
            overwrite = fields[-1] == flag
            if overwrite:
                fields = fields[:-1]
            elif len(fields) == 3:
                fields = [fields[0] + " " + fields[1], fields[2]]
            if len(fields) != 2 or not fields[1].lstrip("-").isdigit():
                raise ValueError("Incorrect dictionary format, expected '<token> <cnt> [flags]'")
            symbol, count = fields[0], int(fields[1])
            if symbol in self.indices and not overwrite:
                raise RuntimeError(f"Duplicate word found when loading Dictionary: '{symbol}'")
            self.add_symbol(symbol, n=count, overwrite=overwrite)

    def save(self, f):
        if isinstance(f, str):
            os.makedirs(os.path.dirname(f) or ".", exist_ok=True)
            with open(f, "w", encoding="utf-8") as fd:
                return self.save(fd)
        for sym, cnt in zip(self.symbols[self.nspecial:], self.count[self.nspecial:]):
            print(f"{sym} {cnt}", file=f)

    def dummy_sentence(self, length: int) -> torch.Tensor:
        t = torch.Tensor(length).uniform_(self.nspecial + 1, len(self)).long()
        t[-1] = self.eos()
        return t

    def encode_line(self, line: str, line_tokenizer=None, add_if_not_exist=True, consumer=None, append_eos=True,
                    reverse_order=False) -> torch.IntTensor:
        """Ids of the words of ``line`` (split by ``line_tokenizer``, default: on whitespace), optionally reversed
        and followed by end-of-sentence.  Unknown words are added or mapped to ``<unk>``; ``consumer(word, id)`` sees
        every word."""
        from metaseq_b200.utils import tokenize_line

        words = list((line_tokenizer or tokenize_line)(line))
        if reverse_order:
            words.reverse()
        lookup = self.add_symbol if add_if_not_exist else self.index
        ids = []
        for word in words:
            ids.append(lookup(word))
            if consumer is not None:
                consumer(word, ids[-1])
        if append_eos:
            ids.append(self.eos_index)
        return torch.tensor(ids, dtype=torch.int32)

    @staticmethod
    def _count_words_in_chunk(filename: str, tokenize, eos_word: str, start: int, end: int) -> Counter:
        from metaseq_b200.file_chunker_utils import Chunker

        counts: Counter = Counter()
        with Chunker(filename, start, end) as lines:
            for line in lines:
                counts.update(tokenize(line))
                counts[eos_word] += 1
        return counts

    @staticmethod
    def add_file_to_dictionary(filename: str, dict: "Dictionary", tokenize, num_workers: int = 1) -> None:
        """Counts the words of a text file (one end-of-sentence symbol per line) into ``dict``.  The file is cut
        at line boundaries into ``num_workers`` byte ranges that are counted by a process pool; symbols are added
        in sorted order per range, so the result does not depend on scheduling (reference:
        metaseq/data/dictionary.py:320-380)."""
        from metaseq_b200.file_chunker_utils import find_offsets
        from metaseq_b200.file_io import PathManager

        local = PathManager.get_local_path(filename)
        offsets = find_offsets(local, max(1, num_workers))
        ranges = list(zip(offsets, offsets[1:]))
        if num_workers > 1:
            from multiprocessing import Pool

            with Pool(processes=num_workers) as pool:
                parts = pool.starmap(Dictionary._count_words_in_chunk,
                                     [(local, tokenize, dict.eos_word, a, b) for a, b in ranges])
        else:
            parts = [Dictionary._count_words_in_chunk(local, tokenize, dict.eos_word, a, b) for a, b in ranges]
        for counts in parts:
            for word, n in sorted(counts.items()):
                dict.add_symbol(word, n)

    @classmethod
    def synthetic(cls, vocab_size: int) -> "Dictionary":
        """Dictionary with ``vocab_size`` entries (4 specials + numbered words), for tasks that
        train on synthetic token ids."""
        d = cls()
        for i in range(vocab_size - d.nspecial):
            d.add_symbol(f"w{i}")
        return d



class TruncatedDictionary:
    """The first ``length`` entries of a dictionary: everything else of the wrapped dictionary (symbols, special
    indices, encoding) is shared, larger indices read as the unknown symbol (metaseq/data/dictionary.py:382-399)."""

    def __init__(self, wrapped_dict, length: int):
        # become a subclass of the wrapped dictionary's class so that isinstance checks and its methods keep working
        self.__class__ = type(wrapped_dict.__class__.__name__, (self.__class__, wrapped_dict.__class__), {})
        self.__dict__ = wrapped_dict.__dict__
        self.wrapped_dict = wrapped_dict
        self.length = min(len(self.wrapped_dict), length)

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        return self.wrapped_dict[i] if i < self.length else self.wrapped_dict.unk()
