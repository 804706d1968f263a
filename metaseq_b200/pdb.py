"""``pdb`` that works inside worker processes started by ``multiprocessing`` (stdin is re-opened from the
parent's descriptor and only one process at a time holds the prompt) and a rank-0-only variant
(reference: metaseq/pdb.py)."""
from __future__ import annotations

import multiprocessing
import os
import pdb
import sys

__all__ = ["set_trace", "set_trace_rank0"]

_stdin = [None]
_stdin_lock = multiprocessing.Lock()
try:
    _stdin_fd = sys.stdin.fileno()
except Exception:  # noqa: BLE001 - no usable stdin (daemon, notebook)
    _stdin_fd = None


class MultiprocessingPdb(pdb.Pdb):
    def __init__(self):
        pdb.Pdb.__init__(self, nosigint=True)

    def _cmdloop(self):
        saved = sys.stdin
        with _stdin_lock:
            try:
                if _stdin_fd is not None:
                    if not _stdin[0]:
                        _stdin[0] = os.fdopen(_stdin_fd)
                    sys.stdin = _stdin[0]
                self.cmdloop()
            finally:
                sys.stdin = saved


def set_trace():
    MultiprocessingPdb().set_trace(sys._getframe().f_back)


def set_trace_rank0():
    """Breaks on global rank 0 only; the other ranks wait at a barrier until it continues."""
    import torch.distributed as dist

    ready = dist.is_available() and dist.is_initialized()
    if not ready or dist.get_rank() == 0:
        MultiprocessingPdb().set_trace(sys._getframe().f_back)
    if ready:
        dist.barrier()
