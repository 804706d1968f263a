"""Path manager with pluggable storage handlers keyed by URI prefix (the role of the reference's iopath-style
``metaseq/file_io/common/__init__.py``: handler interface :94-470, local handler :471-700, manager :702-1246).

The manager picks the handler with the longest matching prefix and falls back to the local file system.  Handler
specific keyword arguments pass through the manager's calls; a handler rejects (strict mode, the default) or only
warns about the ones it does not know.  A copy between two different handlers goes through a local file."""
from __future__ import annotations

import errno
import logging
import os
import shutil
from typing import IO, Any, Dict, List, Optional, Union

logger = logging.getLogger(__name__)


class PathHandler:
    """Operations a storage backend has to provide."""

    _strict_kwargs_check = True

    def _check_kwargs(self, kwargs: Dict[str, Any]) -> None:
        """Keyword arguments that reached a handler which has no use for them: an error in strict mode, a warning
        otherwise."""
        if not kwargs:
            return
        if self._strict_kwargs_check:
            raise ValueError(f"{type(self).__name__} got unused arguments: {sorted(kwargs)}")
        for k, v in kwargs.items():
            logger.warning(f"{type(self).__name__} ignores argument {k}={v!r}")

    def _get_supported_prefixes(self) -> List[str]:
        raise NotImplementedError

    def _mv(self, src: str, dst: str, **kw) -> bool:
        raise NotImplementedError

    def _set_cwd(self, path: Optional[str], **kw) -> bool:
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
    """The local file system.  Relative paths are taken under the handler's working directory when one is set."""

    _cwd: Optional[str] = None

    def _get_supported_prefixes(self):
        return [""]

    def _abs(self, path):
        path = os.fspath(path)
        return path if self._cwd is None or os.path.isabs(path) else os.path.normpath(os.path.join(self._cwd, path))

    def _set_cwd(self, path, **kw):
        self._check_kwargs(kw)
        if path is None:
            self._cwd = None
            return True
        if not os.path.isabs(path) or not os.path.isdir(path):
            logger.error(f"{path} is not an existing absolute directory")
            return False
        self._cwd = path
        return True

    def _get_local_path(self, path, force: bool = False, **kw):
        self._check_kwargs(kw)
        return self._abs(path)

    def _open(self, path, mode="r", buffering=-1, encoding=None, errors=None, newline=None, closefd=True,
              opener=None, **kw):
        self._check_kwargs(kw)
        return open(self._abs(path), mode, buffering=buffering, encoding=encoding, errors=errors, newline=newline,
                    closefd=closefd, opener=opener)

    def _mv(self, src, dst, **kw):
        self._check_kwargs(kw)
        src, dst = self._abs(src), self._abs(dst)
        if os.path.exists(dst):
            logger.error(f"Destination file {dst} already exists.")
            return False
        try:
            shutil.move(src, dst)
            return True
        except Exception as e:
            logger.error(f"Error in move operation - {e}")
            return False

    def _copy(self, src, dst, overwrite=False, **kw):
        self._check_kwargs(kw)
        src, dst = self._abs(src), self._abs(dst)
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
        return self._copy(local_path, dst_path, overwrite, **kw)

    def _exists(self, path, **kw):
        self._check_kwargs(kw)
        return os.path.exists(self._abs(path))

    def _isfile(self, path, **kw):
        self._check_kwargs(kw)
        return os.path.isfile(self._abs(path))

    def _isdir(self, path, **kw):
        self._check_kwargs(kw)
        return os.path.isdir(self._abs(path))

    def _islink(self, path, **kw):
        return os.path.islink(self._abs(path))

    def _ls(self, path, **kw):
        self._check_kwargs(kw)
        return os.listdir(self._abs(path))

    def _mkdirs(self, path, **kw):
        self._check_kwargs(kw)
        try:
            os.makedirs(self._abs(path), exist_ok=True)
        except OSError as e:
            if e.errno != errno.EEXIST:
                raise

    def _rm(self, path, **kw):
        self._check_kwargs(kw)
        os.remove(self._abs(path))

    def _rename(self, src, dst, **kw):
        os.replace(self._abs(src), self._abs(dst))
        return True

    def _symlink(self, src, dst, **kw):
        self._check_kwargs(kw)
        src, dst = self._abs(src), self._abs(dst)
        if os.path.lexists(dst):
            os.remove(dst)
        os.symlink(src, dst)
        return True


class PathManagerBase:
    def __init__(self):
        self._handlers: Dict[str, PathHandler] = {}
        self._native = NativePathHandler()
        self._nb = None
        self._nb_buffered = None
        self._cwd: Optional[str] = None
        self._enable_logging = True

    # ------------------------------------------------------------- handlers
    def register_handler(self, handler: PathHandler, allow_override: bool = True):
        """Registers ``handler`` for its prefixes.  A ``NativePathHandler`` replaces the built-in local handler."""
        assert isinstance(handler, PathHandler), handler
        if isinstance(handler, NativePathHandler):
            if not allow_override:
                raise ValueError("a local-file handler is registered by default; pass allow_override=True to replace it")
            self._native = handler
            return
        for prefix in handler._get_supported_prefixes():
            old = self._handlers.get(prefix)
            if old is not None and not allow_override:
                raise KeyError(f"prefix {prefix} already registered by {type(old).__name__}")
            if old is not None and type(old) is not type(handler):
                logger.warning(f"prefix {prefix!r}: {type(handler).__name__} replaces {type(old).__name__}")
            self._handlers[prefix] = handler

    def _handler(self, path) -> PathHandler:
        path = os.fspath(path)
        for prefix in sorted(self._handlers, key=len, reverse=True):
            if prefix and path.startswith(prefix):
                return self._handlers[prefix]
        return self._native

    def path_requires_pathmanager(self, path) -> bool:
        """True when a non-local handler serves ``path``."""
        return self._handler(path) is not self._native

    def set_strict_kwargs_checking(self, enable: bool) -> None:
        """Strict (default): an argument that a handler does not use raises ``ValueError``; otherwise it warns."""
        self._native._strict_kwargs_check = enable
        for h in self._handlers.values():
            h._strict_kwargs_check = enable

    def set_logging(self, enable_logging: bool = True) -> None:
        self._enable_logging = enable_logging

    def set_cwd(self, path: Optional[str], **kw) -> bool:
        """Working directory that the handler of ``path`` puts in front of relative paths; ``None`` clears it."""
        if path is None and self._cwd is None:
            return True
        if self._handler(path or self._cwd)._set_cwd(path, **kw):
            self._cwd = path
            return True
        return False

    # ------------------------------------------------------------------ I/O
    def open(self, path, mode="r", buffering=-1, encoding=None, errors=None, newline=None, **kw):
        return self._handler(path)._open(path, mode, buffering=buffering, encoding=encoding, errors=errors,
                                         newline=newline, **kw)

    def opena(self, path, mode="a", callback_after_file_close=None, buffering=-1, **kw):
        """Non-blocking write handle: writes are queued to the path's background thread, in order, also across
        handles on the same path.  ``buffering`` > 0 collects writes into chunks of that many bytes first."""
        from .non_blocking_io import NonBlockingIOManager

        key = os.path.normpath(path) if "://" not in str(path) else str(path)
        io_obj = self._handler(path)._open(path, mode, **kw)
        if buffering is not None and buffering > 0:
            if self._nb_buffered is None:
                self._nb_buffered = NonBlockingIOManager(buffered=True)
            return self._nb_buffered.get_non_blocking_io(key, io_obj, callback_after_file_close, buffering)
        if self._nb is None:
            self._nb = NonBlockingIOManager()
        return self._nb.get_non_blocking_io(key, io_obj, callback_after_file_close)

    def async_join(self, *paths):
        """Waits for the queued writes of ``paths`` (all if none is named); re-raises a failed write's exception."""
        ok = True
        for mgr in (self._nb, self._nb_buffered):
            if mgr is None:
                continue
            keys = [os.path.normpath(p) if "://" not in str(p) else str(p) for p in paths]
            mine = [k for k in keys if k in mgr._paths]
            if paths and not mine:
                continue
            ok = mgr._join(*mine) and ok
        return ok

    def async_close(self):
        ok = True
        for mgr in (self._nb, self._nb_buffered):
            if mgr is not None:
                ok = mgr._close_thread_pool() and ok
        return ok

    def copy(self, src, dst, overwrite=False, **kw):
        hs, hd = self._handler(src), self._handler(dst)
        if hs is not hd:
            return self._copy_across_handlers(src, dst, overwrite, **kw)
        return hs._copy(src, dst, overwrite, **kw)

    def _copy_across_handlers(self, src, dst, overwrite, **kw):
        """Source and destination live in different stores: fetch to a local file, then upload."""
        local = self._handler(src)._get_local_path(src, **kw)
        return self._handler(dst)._copy_from_local(local, dst, overwrite=overwrite, **kw)

    def mv(self, src, dst, **kw):
        hs, hd = self._handler(src), self._handler(dst)
        assert hs is hd, "source and destination must be served by the same handler"
        return hs._mv(src, dst, **kw)

    def copy_from_local(self, local_path, dst_path, overwrite=False, **kw):
        assert os.path.exists(local_path), f"local path {local_path} does not exist"
        return self._handler(dst_path)._copy_from_local(local_path, dst_path, overwrite, **kw)

    def get_local_path(self, path, force: bool = False, **kw):
        path = os.fspath(path)
        return self._handler(path)._get_local_path(path, force=force, **kw)

    def exists(self, path, **kw):
        return self._handler(path)._exists(path, **kw)

    def isfile(self, path, **kw):
        return self._handler(path)._isfile(path, **kw)

    def isdir(self, path, **kw):
        return self._handler(path)._isdir(path, **kw)

    def islink(self, path):
        return self._handler(path)._islink(path)

    def ls(self, path, **kw):
        return self._handler(path)._ls(path, **kw)

    def mkdirs(self, path, **kw):
        return self._handler(path)._mkdirs(path, **kw)

    def rm(self, path, **kw):
        return self._handler(path)._rm(path, **kw)

    def rename(self, src, dst):
        if not self.supports_rename(src):
            raise ValueError(f"{src} is served by {type(self._handler(src)).__name__}, which cannot rename")
        return self._handler(src)._rename(src, dst)

    def symlink(self, src, dst, **kw):
        assert self._handler(src) is self._handler(dst), "source and destination must be served by the same handler"
        return self._handler(src)._symlink(src, dst, **kw)

    def chmod(self, path, mode):
        if self._handler(path) is self._native:
            os.chmod(self._native._abs(path), mode)

    def supports_rename(self, path):
        return self._handler(path) is self._native
