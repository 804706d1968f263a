"""Splitting a text file into byte ranges that start on line boundaries, for parallel preprocessing
(reference: metaseq/file_chunker_utils.py)."""
from __future__ import annotations

import os
import typing as tp


def _safe_readline(fd) -> str:
    """``readline`` that steps back when the seek landed inside a multi-byte character."""
    pos = fd.tell()
    while True:
        try:
            return fd.readline()
        except UnicodeDecodeError:
            pos -= 1
            fd.seek(pos)


def find_offsets(filename: str, num_chunks: int) -> tp.List[int]:
    """``num_chunks + 1`` byte offsets; chunk i is ``[offsets[i], offsets[i+1])`` and starts at a line start."""
    with open(filename, "r", encoding="utf-8") as f:
        size = os.fstat(f.fileno()).st_size
        step = size // num_chunks
        offsets = [0] * (num_chunks + 1)
        for i in range(1, num_chunks):
            f.seek(step * i)
            _safe_readline(f)  # finish the line the seek landed in
            offsets[i] = f.tell()
        offsets[-1] = size
        return offsets


class ChunkLineIterator:
    """Lines of ``fd`` between two offsets."""

    def __init__(self, fd, start_offset: int, end_offset: int):
        self._fd, self._start, self._end = fd, start_offset, end_offset

    def __iter__(self) -> tp.Iterable[str]:
        self._fd.seek(self._start)
        line = _safe_readline(self._fd)
        while line:
            pos = self._fd.tell()
            # some file systems report positions beyond 2**32 with a spurious high bit; ignore those
            if self._end > 0 and pos > self._end and pos < self._end + 2 ** 32:
                break
            yield line
            line = self._fd.readline()


class Chunker:
    """Context manager yielding a ``ChunkLineIterator`` over ``path[start_offset:end_offset]``."""

    def __init__(self, path: str, start_offset: int, end_offset: int):
        self.path, self.start_offset, self.end_offset = path, start_offset, end_offset

    def __enter__(self) -> ChunkLineIterator:
        self.fd = open(self.path, "r", encoding="utf-8")
        return ChunkLineIterator(self.fd, self.start_offset, self.end_offset)

    def __exit__(self, exc_type, exc_val, exc_tb) -> None:
        self.fd.close()
