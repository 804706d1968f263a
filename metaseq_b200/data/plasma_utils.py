"""Sharing large read-only numpy arrays between data-loader workers.

The reference keeps them in an Apache Arrow plasma store (metaseq/data/plasma_utils.py); plasma has been
removed from pyarrow, so here the array lives in a POSIX shared-memory segment (``multiprocessing.shared_memory``):
the creating process copies the array in once, pickling ships only the segment name, and every worker maps
the same pages.  ``PlasmaArray`` / ``PlasmaView`` keep the reference's names and call signatures."""
from __future__ import annotations

import hashlib
import json
from multiprocessing import shared_memory
from typing import Hashable

import numpy as np


class PlasmaArray:
    """Wraps an array; after pickling the copy reads from shared memory.  Arrays under 1 MB are pickled by value."""

    def __init__(self, array):
        self._array = array
        self.disable = array.nbytes < 134217728 // 128
        self._shm = None
        self._meta = None

    @property
    def array(self):
        if self._array is None and self._meta is not None:
            name, shape, dtype = self._meta
            self._shm = shared_memory.SharedMemory(name=name)
            self._array = np.ndarray(shape, dtype=np.dtype(dtype), buffer=self._shm.buf)
        return self._array

    @property
    def plasma(self):
        """The sharing backend (the shared-memory module), or ``None`` when this array is small enough to be
        pickled by value.  Named after the reference's store."""
        return None if self.disable else shared_memory

    def start_server(self):
        """Publishes the array: creates the segment and copies the data in (there is no server process; the
        kernel keeps the pages).  Called on first pickling; calling it again does nothing."""
        if self.plasma is None or self._meta is not None:
            return
        shm = shared_memory.SharedMemory(create=True, size=max(1, self._array.nbytes))
        view = np.ndarray(self._array.shape, dtype=self._array.dtype, buffer=shm.buf)
        view[...] = self._array
        self._owner = shm
        self._meta = (shm.name, self._array.shape, self._array.dtype.str)

    @property
    def client(self):
        """This process's attachment to the segment (``None`` before the array is published)."""
        if self._meta is None:
            return None
        owner = getattr(self, "_owner", None)
        if owner is not None:
            return owner
        if self._shm is None:
            self._shm = shared_memory.SharedMemory(name=self._meta[0])
        return self._shm

    def __getstate__(self):
        if self.disable:
            return {"array": self._array, "meta": None}
        self.start_server()
        return {"array": None, "meta": self._meta}

    def __setstate__(self, state):
        self._array = state["array"]
        self._meta = state["meta"]
        self.disable = self._meta is None
        self._shm = None

    def __del__(self):
        owner = getattr(self, "_owner", None)
        if owner is not None:
            try:
                owner.close()
                owner.unlink()
            except Exception:  # noqa: BLE001
                pass
        elif getattr(self, "_shm", None) is not None:
            try:
                self._shm.close()
            except Exception:  # noqa: BLE001
                pass


class PlasmaView:
    """Array stored under a name derived from ``(split_path, hash_data)`` so that independent processes that
    build the same view attach to one segment instead of each holding a copy."""

    def __init__(self, array, split_path: str, hash_data: Hashable, plasma_path=None):
        assert split_path is not None
        self.split_path = split_path
        self.name = self.get_object_id(split_path, hash_data)
        self._shape, self._dtype = array.shape, array.dtype.str
        self._owner = None
        try:
            shm = shared_memory.SharedMemory(name=self.name, create=True, size=max(1, array.nbytes))
            np.ndarray(array.shape, dtype=array.dtype, buffer=shm.buf)[...] = array
            self._owner = shm
            self._shm = shm
        except FileExistsError:
            self._shm = shared_memory.SharedMemory(name=self.name)

    @property
    def array(self):
        if self._shm is None:
            self._shm = shared_memory.SharedMemory(name=self.name)
        return np.ndarray(self._shape, dtype=np.dtype(self._dtype), buffer=self._shm.buf)

    @property
    def client(self):
        """This process's attachment to the segment."""
        if self._shm is None:
            self._shm = shared_memory.SharedMemory(name=self.name)
        return self._shm

    @staticmethod
    def get_object_id(split_path: str, hash_data: Hashable) -> str:
        h = hashlib.blake2b(bytes(split_path, "utf-8"), digest_size=10)
        h.update(json.dumps(hash_data).encode("utf-8"))
        return "msq_" + h.hexdigest()

    def __getstate__(self):
        state = self.__dict__.copy()
        state["_shm"] = None
        state["_owner"] = None
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)

    def disconnect(self):
        if self._shm is not None:
            self._shm.close()
            self._shm = None

    def __del__(self):
        try:
            if self._owner is not None:
                self._owner.close()
                self._owner.unlink()
            elif self._shm is not None:
                self._shm.close()
        except Exception:  # noqa: BLE001
            pass

    def __len__(self):
        return len(self.array)


class PlasmaStore:
    """Owner of the shared segments of a job.  The reference starts a ``plasma_store`` server process here
    (metaseq/data/plasma_utils.py:182-196); shared memory needs no server, so this object only remembers the
    segments registered with it and unlinks them in ``close()`` (or when it is collected)."""

    def __init__(self, path: str = "/tmp/plasma", nbytes: int = 0):
        self.path, self.nbytes = path, nbytes
        self._segments = []
        self.server = None  # no process to manage

    @staticmethod
    def start(path: str = "/tmp/plasma", nbytes: int = 0) -> None:
        return None

    def register(self, segment: shared_memory.SharedMemory) -> shared_memory.SharedMemory:
        self._segments.append(segment)
        return segment

    def close(self) -> None:
        for seg in self._segments:
            try:
                seg.close()
                seg.unlink()
            except FileNotFoundError:
                pass
        self._segments = []

    def __del__(self):
        self.close()
