"""Write-behind file handles.

``write`` only enqueues; one worker thread per *path* runs the queued operations in the order they were
issued, also across several handles opened on the same path; ``close`` queues the real close and an optional
callback (an upload, a rename) behind the writes.  ``NonBlockingBufferedIO`` additionally collects small writes
into buffers of ``buffering`` bytes so that each queued operation is one large write.  The manager joins the
workers of some or all paths and remembers the first exception of a failed operation, which the join calls
re-raise (reference: metaseq/file_io/common/non_blocking_io.py).
"""
from __future__ import annotations

import io
import logging
import threading
from dataclasses import dataclass
from queue import Queue
from typing import IO, Callable, Dict, List, Optional, Union

logger = logging.getLogger(__name__)

_JOIN_SECONDS = 600


@dataclass
class PathData:
    """The ordered job queue of one path and the thread that drains it."""

    queue: Queue
    thread: threading.Thread


class NonBlockingIO(io.IOBase):
    """Every operation is handed to ``notify_manager`` as a callable; nothing touches the file on this thread."""

    def __init__(self, notify_manager: Callable[[Callable[[], None]], None], io_obj: IO,
                 callback_after_file_close: Optional[Callable[[], None]] = None):
        super().__init__()
        self._notify = notify_manager
        self._io = io_obj
        self._callback = callback_after_file_close
        self._close_called = False

    def readable(self) -> bool:
        return False

    def writable(self) -> bool:
        return True

    def seekable(self) -> bool:
        return True

    def write(self, b: Union[bytes, bytearray, str]) -> None:
        self._notify(lambda: self._io.write(b))

    def seek(self, offset: int, whence: int = 0):
        self._notify(lambda: self._io.seek(offset, whence))

    def tell(self):
        raise ValueError("ioPath async writes does not support `tell` calls.")

    def truncate(self, size: Optional[int] = None):
        self._notify(lambda: self._io.truncate(0 if size is None else size))

    def flush(self) -> None:
        pass  # the queued close flushes; there is nothing buffered on this side

    def _finish(self):
        self._io.close()
        if self._callback is not None:
            self._callback()

    def close(self) -> None:
        if self._close_called:
            return
        self._close_called = True
        self._notify(self._finish)


class NonBlockingBufferedIO(NonBlockingIO):
    """Collects writes until ``buffering`` bytes are pending (or ``flush`` / ``close``), then queues them as one
    write (text stays text, bytes stay bytes: the underlying file decides which it takes)."""

    MAX_BUFFER_BYTES = 10 * 1024 * 1024

    def __init__(self, notify_manager, io_obj: IO, callback_after_file_close=None, buffering: int = -1):
        super().__init__(notify_manager, io_obj, callback_after_file_close)
        self._limit = buffering if buffering and buffering > 0 else self.MAX_BUFFER_BYTES
        self._pending: List[Union[bytes, str]] = []
        self._pending_bytes = 0

    def write(self, b: Union[bytes, bytearray, str]) -> None:
        piece = bytes(b) if isinstance(b, (bytearray, memoryview)) else b
        self._pending.append(piece)
        self._pending_bytes += len(piece)
        if self._pending_bytes >= self._limit:
            self.flush()

    def flush(self) -> None:
        if not self._pending:
            return
        pieces, self._pending, self._pending_bytes = self._pending, [], 0
        joined = (b"" if isinstance(pieces[0], bytes) else "").join(pieces)
        self._notify(lambda: self._io.write(joined))

    def seek(self, offset: int, whence: int = 0):
        self.flush()
        super().seek(offset, whence)

    def truncate(self, size: Optional[int] = None):
        self.flush()
        super().truncate(size)

    def close(self) -> None:
        if not self._close_called:
            self.flush()
        super().close()


class NonBlockingIOManager:
    def __init__(self, buffered: bool = False):
        self._buffered = bool(buffered)
        self._paths: Dict[str, PathData] = {}
        self._lock = threading.Lock()
        self._error: Optional[BaseException] = None

    # ------------------------------------------------------------- workers
    def _drain(self, path: str, queue: Queue) -> None:
        while True:
            job = queue.get()
            if job is None:
                return
            try:
                job()
            except BaseException as e:  # noqa: BLE001 - keep draining so a later close still runs
                logger.error(f"async write to {path} failed: {e}")
                if self._error is None:
                    self._error = e

    def _submit(self, path: str, job: Optional[Callable[[], None]]) -> None:
        """Queues ``job`` for ``path`` (starting the path's worker if it has none).  Taking the lock for the put
        keeps a job from landing behind the stop marker of a concurrent join."""
        with self._lock:
            data = self._paths.get(path)
            if data is None:
                queue: Queue = Queue()
                thread = threading.Thread(target=self._drain, args=(path, queue), daemon=True, name=f"nbio:{path}")
                thread.start()
                data = self._paths[path] = PathData(queue, thread)
            if job is not None:
                data.queue.put(job)

    # ----------------------------------------------------------------- API
    def get_non_blocking_io(self, path: str, io_obj: IO, callback_after_file_close=None, buffering: int = -1):
        if not self._buffered and buffering != -1:
            raise ValueError("NonBlockingIO is not using a buffered writer but `buffering` arg is set to "
                             f"non-default value of {buffering} != -1.")
        self._submit(path, None)

        def submit(job):  # after a join the path gets a fresh worker
            self._submit(path, job)

        if self._buffered:
            return NonBlockingBufferedIO(submit, io_obj, callback_after_file_close, buffering)
        return NonBlockingIO(submit, io_obj, callback_after_file_close)

    def _stop(self, paths) -> bool:
        with self._lock:
            picked = {p: self._paths.pop(p) for p in list(self._paths) if not paths or p in paths}
        ok = True
        for p, data in picked.items():
            data.queue.put(None)  # behind everything queued so far
            data.thread.join(_JOIN_SECONDS)
            ok = ok and not data.thread.is_alive()
        err, self._error = self._error, None
        if err is not None:
            raise err
        return ok

    def _join(self, *paths: str) -> bool:
        """Waits until everything queued so far for ``paths`` (all paths if none is named) has run.  A handle that
        is still open keeps working afterwards: its next operation starts a fresh worker."""
        unknown = [p for p in paths if p not in self._paths]
        if unknown:
            raise ValueError(f"{unknown[0]} has no async IO associated with it. Make sure `opena({unknown[0]})` is "
                             "called first.")
        return self._stop(set(paths))

    def _close_thread_pool(self) -> bool:
        return self._stop(set())
