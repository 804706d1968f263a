"""Memory-mapped JSON-lines dataset with a cached line-offset index.

One JSON document per line.  The byte offset of every line is computed once and
cached next to the file as ``<path>.fairseq.idx.npy`` (the reference's cache
name, so existing caches are reused: metaseq/data/jsonl_dataset.py:55-68); with
several ranks only global rank 0 builds it while the others wait at a barrier.
``epoch`` / ``data_subshard_count`` select every k-th line so that one pass over
the file takes ``data_subshard_count`` epochs (:89-134).
"""
from __future__ import annotations

import json
import logging
import mmap
import os
import threading
from pathlib import Path
from typing import Callable, Optional

import numpy as np
import torch

logger = logging.getLogger(__name__)


class JsonlDataset(torch.utils.data.Dataset):
    def __init__(self, path: str, tokenizer: Optional[Callable] = None, recache: bool = False, epoch: int = 1,
                 data_subshard_count: int = 1):
        self.path = path
        self.tokenizer = tokenizer
        self.threadlocal = threading.local()
        self.epoch = epoch
        self.data_subshard_count = data_subshard_count
        self.cache = Path(f"{path}.fairseq.idx.npy")
        self._build_or_load_index(recache)
        self.offsets = self._subshard_offsets()

    # ---------------------------------------------------------------- index
    def _build_or_load_index(self, recache: bool):
        from metaseq_b200.parallel import utils as dist_utils

        multi = dist_utils.is_initialized() and dist_utils.get_global_world_size() > 1
        if multi and dist_utils.get_global_rank() != 0:
            torch.distributed.barrier()
        if not self.cache.exists() or recache:
            if not multi or dist_utils.get_global_rank() == 0:
                np.save(self.cache, self._scan_offsets(self.path))
        if multi and dist_utils.get_global_rank() == 0:
            torch.distributed.barrier()
        self._all_offsets = np.load(self.cache)
        if len(self._all_offsets) and self._all_offsets[-1] >= max(1, os.path.getsize(self.path)):
            # stale cache from another file of the same name
            self._all_offsets = self._scan_offsets(self.path)
            try:
                np.save(self.cache, self._all_offsets)
            except OSError:
                pass

    @staticmethod
    def _scan_offsets(path: str) -> np.ndarray:
        logger.info(f"Building index for file: {path}")
        offsets = []
        with open(path, "rb") as f:
            pos = 0
            for line in f:
                if line.strip():
                    offsets.append(pos)
                pos += len(line)
        return np.asarray(offsets, dtype=np.int64)

    def _subshard_offsets(self) -> np.ndarray:
        k = self.data_subshard_count
        if k <= 1:
            return self._all_offsets
        which = (self.epoch - 1) % k
        return self._all_offsets[which::k]

    # ----------------------------------------------------------------- access
    def _file(self):
        if not hasattr(self.threadlocal, "handles"):
            f = open(self.path, "rb")
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if os.path.getsize(self.path) > 0 else None
            self.threadlocal.handles = (f, mm)
        return self.threadlocal.handles[1]

    def __getstate__(self):
        d = {k: v for k, v in self.__dict__.items() if k != "threadlocal"}
        return d

    def __setstate__(self, d):
        self.__dict__ = d
        self.threadlocal = threading.local()

    def __del__(self):
        h = getattr(getattr(self, "threadlocal", None), "handles", None)
        if h:
            f, mm = h
            if mm is not None:
                mm.close()
            f.close()

    @staticmethod
    def exists(path):
        return os.path.exists(path)

    def __len__(self):
        return len(self.offsets)

    def __getitem__(self, idx):
        if idx < 0 or idx >= len(self):
            raise IndexError
        mm = self._file()
        mm.seek(int(self.offsets[idx]))
        item = json.loads(mm.readline().decode("utf-8"))
        if self.tokenizer is not None:
            item = self.tokenizer(item)
        return item


if __name__ == "__main__":
    # python -m metaseq_b200.data.jsonl_dataset FILE... : pre-build the index caches
    import sys

    for p in sys.argv[1:]:
        JsonlDataset(p, recache=True)
