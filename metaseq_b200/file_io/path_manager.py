"""Minimal path manager with pluggable handlers keyed by URI prefix."""
from __future__ import annotations

import errno
import logging
import os
import shutil
from typing import IO, Any, Dict, List, Optional, Union

logger = logging.getLogger(__name__)


class PathHandler:
    """Operations a storage backend has to provide."""

    def _get_supported_prefixes(self) -> List[str]:
        raise NotImplementedError

    def _get_local_path(self, path: str, **kw) -> str:
        raise NotImplementedError

    def _open(self, path: str, mode: str = "r", buffering: int = -1, **kw) -> IO[Any]:
        raise NotImplementedError

    def _copy(self, src: str, dst: str, overwrite: bool = False, **kw) -> bool:
        raise NotImplementedError

    def _exists(self, path: str, **kw) -> bool:
        raise NotImplementedError

    def _isfile(self, path: str, **kw) -> bool:
        raise NotImplementedError

    def _isdir(self, path: str, **kw) -> bool:
        raise NotImplementedError

    def _ls(self, path: str, **kw) -> List[str]:
        raise NotImplementedError

    def _mkdirs(self, path: str, **kw) -> None:
        raise NotImplementedError

    def _rm(self, path: str, **kw) -> None:
        raise NotImplementedError

    def _rename(self, src: str, dst: str, **kw) -> bool:
        raise NotImplementedError

    def _symlink(self, src: str, dst: str, **kw) -> bool:
        raise NotImplementedError

    def _islink(self, path: str, **kw) -> bool:
        return False

    def _copy_from_local(self, local_path: str, dst_path: str, overwrite: bool = False, **kw) -> bool:
        raise NotImplementedError


class NativePathHandler(PathHandler):
    def _get_supported_prefixes(self):
        return [""]

    def _get_local_path(self, path, **kw):
        return os.fspath(path)

    def _open(self, path, mode="r", buffering=-1, encoding=None, errors=None, newline=None, **kw):
        return open(path, mode, buffering=buffering, encoding=encoding, errors=errors, newline=newline)

    def _copy(self, src, dst, overwrite=False, **kw):
        if os.path.exists(dst) and not overwrite:
            logger.error(f"Destination file {dst} already exists.")
            return False
        try:
            shutil.copyfile(src, dst)
            return True
        except Exception as e:
            logger.error(f"Error in file copy - {e}")
            return False

    def _copy_from_local(self, local_path, dst_path, overwrite=False, **kw):
        return self._copy(local_path, dst_path, overwrite)

    def _exists(self, path, **kw):
        return os.path.exists(path)

    def _isfile(self, path, **kw):
        return os.path.isfile(path)

    def _isdir(self, path, **kw):
        return os.path.isdir(path)

    def _islink(self, path, **kw):
        return os.path.islink(path)

    def _ls(self, path, **kw):
        return os.listdir(path)

    def _mkdirs(self, path, **kw):
        try:
            os.makedirs(path, exist_ok=True)
        except OSError as e:
            if e.errno != errno.EEXIST:
                raise

    def _rm(self, path, **kw):
        os.remove(path)

    def _rename(self, src, dst, **kw):
        os.replace(src, dst)
        return True

    def _symlink(self, src, dst, **kw):
        if os.path.lexists(dst):
            os.remove(dst)
        os.symlink(src, dst)
        return True


class PathManagerBase:
    def __init__(self):
        self._handlers: Dict[str, PathHandler] = {}
        self._native = NativePathHandler()
        self._nb = None

    def register_handler(self, handler: PathHandler, allow_override: bool = True):
        for prefix in handler._get_supported_prefixes():
            if prefix in self._handlers and not allow_override:
                raise KeyError(f"prefix {prefix} already registered")
            self._handlers[prefix] = handler

    def _handler(self, path) -> PathHandler:
        path = os.fspath(path)
        for prefix in sorted(self._handlers, key=len, reverse=True):
            if prefix and path.startswith(prefix):
                return self._handlers[prefix]
        return self._native

    def open(self, path, mode="r", buffering=-1, encoding=None, errors=None, newline=None):
        return self._handler(path)._open(path, mode, buffering=buffering, encoding=encoding, errors=errors,
                                         newline=newline)

    def opena(self, path, mode="a", callback_after_file_close=None, **kw):
        """Non-blocking write handle: writes are queued to a background thread."""
        if self._nb is None:
            from .non_blocking_io import NonBlockingIOManager

            self._nb = NonBlockingIOManager()
        return self._nb.get_non_blocking_io(path, self._handler(path)._open(path, mode), callback_after_file_close)

    def async_join(self, *paths):
        return self._nb._join(*paths) if self._nb is not None else True

    def async_close(self):
        return self._nb._close_thread_pool() if self._nb is not None else True

    def copy(self, src, dst, overwrite=False):
        return self._handler(src)._copy(src, dst, overwrite)

    def copy_from_local(self, local_path, dst_path, overwrite=False):
        return self._handler(dst_path)._copy_from_local(local_path, dst_path, overwrite)

    def get_local_path(self, path, **kw):
        return self._handler(path)._get_local_path(path, **kw)

    def exists(self, path):
        return self._handler(path)._exists(path)

    def isfile(self, path):
        return self._handler(path)._isfile(path)

    def isdir(self, path):
        return self._handler(path)._isdir(path)

    def islink(self, path):
        return self._handler(path)._islink(path)

    def ls(self, path):
        return self._handler(path)._ls(path)

    def mkdirs(self, path):
        return self._handler(path)._mkdirs(path)

    def rm(self, path):
        return self._handler(path)._rm(path)

    def rename(self, src, dst):
        return self._handler(src)._rename(src, dst)

    def symlink(self, src, dst):
        return self._handler(src)._symlink(src, dst)

    def chmod(self, path, mode):
        if self._handler(path) is self._native:
            os.chmod(path, mode)

    def supports_rename(self, path):
        return self._handler(path) is self._native
