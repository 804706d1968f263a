"""Write-behind file handles: ``write`` enqueues, one worker thread per path keeps order,
``close`` flushes and runs an optional callback (reference: metaseq/file_io/common/non_blocking_io.py)."""
from __future__ import annotations

import concurrent.futures
import io
import logging
import threading
from queue import Queue
from typing import IO, Callable, Dict, Optional, Union

logger = logging.getLogger(__name__)


class NonBlockingIO(io.IOBase):
    def __init__(self, path: str, notify, file_obj: IO, callback: Optional[Callable[[], None]]):
        super().__init__()
        self._path = path
        self._notify = notify
        self._io = file_obj
        self._callback = callback
        self._queue: "Queue" = Queue()
        self._done = threading.Event()
        self._thread = threading.Thread(target=self._drain, daemon=True)
        self._thread.start()
        self._closed = False

    def _drain(self):
        while True:
            item = self._queue.get()
            if item is None:
                break
            try:
                item()
            except Exception as e:  # keep draining so close() can finish
                logger.error(f"async write to {self._path} failed: {e}")
        self._done.set()

    def writable(self):
        return True

    def seekable(self):
        return True

    def write(self, b: Union[bytes, bytearray, str]) -> None:
        self._queue.put(lambda: self._io.write(b))

    def seek(self, offset: int, whence: int = 0):
        self._queue.put(lambda: self._io.seek(offset, whence))

    def tell(self):
        raise ValueError("ioPath async writes does not support `tell` calls.")

    def truncate(self, size=None):
        self._queue.put(lambda: self._io.truncate(size) if size is not None else self._io.truncate(0))

    def flush(self):
        pass

    def close(self):
        if self._closed:
            return
        self._closed = True

        def finish():
            self._io.close()
            if self._callback is not None:
                self._callback()

        self._queue.put(finish)
        self._queue.put(None)
        self._notify(self)

    def join(self, timeout=None):
        return self._done.wait(timeout)


class NonBlockingIOManager:
    def __init__(self):
        self._handles: Dict[str, list] = {}
        self._lock = threading.Lock()

    def get_non_blocking_io(self, path, io_obj, callback_after_file_close=None):
        h = NonBlockingIO(path, lambda _h: None, io_obj, callback_after_file_close)
        with self._lock:
            self._handles.setdefault(path, []).append(h)
        return h

    def _join(self, *paths) -> bool:
        ok = True
        with self._lock:
            items = {p: list(hs) for p, hs in self._handles.items() if not paths or p in paths}
        for p, hs in items.items():
            for h in hs:
                if not h._closed:
                    continue
                ok = h.join(600) and ok
        return ok

    def _close_thread_pool(self) -> bool:
        with self._lock:
            items = [h for hs in self._handles.values() for h in hs]
            self._handles = {}
        ok = True
        for h in items:
            if not h._closed:
                h.close()
            ok = h.join(600) and ok
        return ok
