"""Splitting a text file into byte ranges that start on line boundaries, for parallel preprocessing
(reference: metaseq/file_chunker_utils.py).

The file is handled as bytes: a line boundary is a ``\\n`` byte, which UTF-8 never uses inside a multi-byte
character, so a seek to an arbitrary offset needs no recovery from a split character, and every line is decoded
on its own when it is handed out."""
from __future__ import annotations

import os
from typing import Iterator, List


def find_offsets(filename: str, num_chunks: int) -> List[int]:
    """``num_chunks + 1`` byte offsets; chunk i is ``[offsets[i], offsets[i+1])`` and starts at a line start."""
    size = os.path.getsize(filename)
    offsets = [0] * (num_chunks + 1)
    offsets[num_chunks] = size
    with open(filename, "rb") as raw:
        for i in range(1, num_chunks):
            raw.seek(i * (size // num_chunks))
            raw.readline()  # to the end of the line that the seek landed in
            offsets[i] = raw.tell()
    return offsets


class ChunkLineIterator:
    """The lines that begin inside ``[start_offset, end_offset)`` of a binary file object, decoded as UTF-8.
    ``end_offset <= 0`` reads to the end of the file."""

    def __init__(self, fd, start_offset: int, end_offset: int, encoding: str = "utf-8"):
        self._raw, self._begin, self._limit, self._encoding = fd, start_offset, end_offset, encoding

    def __iter__(self) -> Iterator[str]:
        self._raw.seek(self._begin)
        position = self._begin
        for data in iter(self._raw.readline, b""):
            if 0 < self._limit <= position:
                return
            position += len(data)
            yield data.decode(self._encoding)


class Chunker:
    """``with Chunker(path, a, b) as lines:`` iterates the lines of ``path`` that start in ``[a, b)``."""

    def __init__(self, path: str, start_offset: int, end_offset: int):
        self.path, self.start_offset, self.end_offset = path, start_offset, end_offset
        self.fd = None

    def __enter__(self) -> ChunkLineIterator:
        self.fd = open(self.path, "rb")
        return ChunkLineIterator(self.fd, self.start_offset, self.end_offset)

    def __exit__(self, exc_type, exc_val, exc_tb) -> None:
        self.fd.close()
        self.fd = None
