"""Path abstraction: local paths natively, ``s3://`` and Azure blob URLs through optional
handlers when their SDKs are installed (reference: metaseq/file_io/__init__.py:11-64 and the
iopath-style manager in metaseq/file_io/common/)."""
from __future__ import annotations

import logging
import os
import shutil
from typing import IO, Any, Callable, Dict, List, Optional

import torch

from .path_manager import NativePathHandler, PathHandler, PathManagerBase
from .non_blocking_io import NonBlockingIOManager  # noqa: F401

logger = logging.getLogger(__name__)

PathManager = PathManagerBase()

from .s3 import S3PathHandler  # noqa: E402  (boto3 is imported on first use of an s3:// path)

PathManager.register_handler(S3PathHandler())
from .azure_blob import AzureBlobPathHandler  # noqa: E402  (the SDK is imported on first use of an az:// path)

PathManager.register_handler(AzureBlobPathHandler())


def recursively_cast_dictconfigs(cfg):
    """Config nodes saved by other tools (mapping-like objects) become plain dicts."""
    if isinstance(cfg, dict):
        return {k: recursively_cast_dictconfigs(v) for k, v in cfg.items()}
    if hasattr(cfg, "items") and not isinstance(cfg, dict) and cfg.__class__.__name__ == "DictConfig":
        return {k: recursively_cast_dictconfigs(v) for k, v in cfg.items()}
    return cfg


def torch_load_cpu(path):
    with PathManager.open(path, "rb") as f:
        state = torch.load(f, map_location=torch.device("cpu"), weights_only=False)
    if isinstance(state, dict) and "cfg" in state:
        state["cfg"] = recursively_cast_dictconfigs(state["cfg"])
        if isinstance(state["cfg"], dict) and state["cfg"].get("model") is not None \
                and isinstance(state["cfg"]["model"], dict) and "arch" in state["cfg"]["model"] and False:
            pass
    return state


def load_and_pop_last_optimizer_state(pth):
    st = torch_load_cpu(pth)
    st.pop("last_optimizer_state", None)
    return st


def get_cache_dir(cache_dir: Optional[str] = None) -> str:
    """Directory for local copies of remote files: the argument, else ``$FVCORE_CACHE``, else
    ``~/.torch/iopath_cache``; a directory under the system's temporary folder when that one cannot be written
    (metaseq/file_io/common/__init__.py:35-59)."""
    import tempfile

    if cache_dir is None:
        cache_dir = os.path.expanduser(os.getenv("FVCORE_CACHE", "~/.torch/iopath_cache"))
    try:
        os.makedirs(cache_dir, exist_ok=True)
        if not os.access(cache_dir, os.W_OK):
            raise OSError(f"{cache_dir} is not writable")
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), "iopath_cache")
        logger.warning(f"{cache_dir} is not accessible! Using {fallback} instead!")
        os.makedirs(fallback, exist_ok=True)
        cache_dir = fallback
    return cache_dir


class file_lock:
    """``with file_lock(path):`` holds an exclusive advisory lock on ``path + ".lock"`` so that several workers do
    not download or build the same file at once; waiting gives up with ``TimeoutError`` after ``timeout`` seconds
    (metaseq/file_io/common/__init__.py:62-91, which uses ``portalocker`` for the same purpose)."""

    def __init__(self, path: str, timeout: float = 1800.0, poll: float = 0.05):
        self.lock_path, self.timeout, self.poll = path + ".lock", timeout, poll
        self._fh = None

    def __enter__(self):
        import fcntl
        import time

        os.makedirs(os.path.dirname(os.path.abspath(self.lock_path)), exist_ok=True)
        self._fh = open(self.lock_path, "a+")
        deadline = time.monotonic() + self.timeout
        while True:
            try:
                fcntl.flock(self._fh.fileno(), fcntl.LOCK_EX | fcntl.LOCK_NB)
                return self
            except OSError:
                if time.monotonic() >= deadline:
                    self._fh.close()
                    self._fh = None
                    raise TimeoutError(f"could not lock {self.lock_path} within {self.timeout} s")
                time.sleep(self.poll)

    def __exit__(self, *exc):
        import fcntl

        if self._fh is not None:
            fcntl.flock(self._fh.fileno(), fcntl.LOCK_UN)
            self._fh.close()
            self._fh = None
        return False
