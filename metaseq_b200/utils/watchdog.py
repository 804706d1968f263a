"""Host-side watchdog for a training or serving loop.

The device side of failure detection is the bounded wait: a kernel that gives up on a peer leaves a code in
the status word and returns (``csrc/sm100_common.cuh``).  This is the host side: a daemon thread that notices
when the loop has stopped making progress (no heartbeat, or a CUDA event that never completes: a lost peer, a
stuck collective, a wedged data loader), reports where every thread is, and hands control to a callback: by
default it interrupts the main thread so that the usual exception path (checkpoint-on-exit, process-group
teardown, SLURM requeue) runs.  It also polls the kernel status word, so that a timed-out wait is reported at
once instead of at the next host synchronisation.

The reference has no such component: it relies on ``NCCL_ASYNC_ERROR_HANDLING`` and on the scheduler's
requeue (metaseq/launcher/slurm.py:150, :269-273).
"""
from __future__ import annotations

import faulthandler
import logging
import sys
import threading
import time
from typing import Callable, Optional

logger = logging.getLogger(__name__)


class StepWatchdog:
    """``beat()`` once per step; ``timeout_s`` without a beat (or with a watched CUDA event still pending, or
    a non-zero kernel status word) fires ``on_timeout(reason)`` once and stops the watchdog.

    ``status_fn`` returns the kernel status word (0 = healthy) without clearing it; ``None`` disables that
    check.  ``on_timeout`` defaults to dumping all thread stacks and interrupting the main thread."""

    def __init__(self, timeout_s: float, on_timeout: Optional[Callable[[str], None]] = None, poll_s: float = 1.0,
                 status_fn: Optional[Callable[[], int]] = None):
        assert timeout_s > 0
        self.timeout_s = float(timeout_s)
        self.poll_s = min(float(poll_s), self.timeout_s / 2)
        self.on_timeout = on_timeout or self._interrupt_main
        self.status_fn = status_fn
        self._last = time.monotonic()
        self._event = None
        self._event_since = 0.0
        self._stop = threading.Event()
        self._lock = threading.Lock()
        self.fired: Optional[str] = None
        self._thread = threading.Thread(target=self._run, name="msq-watchdog", daemon=True)

    # ---------------------------------------------------------------- control
    def start(self) -> "StepWatchdog":
        self._last = time.monotonic()
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread.is_alive() and threading.current_thread() is not self._thread:
            self._thread.join(timeout=5 * self.poll_s + 1)

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
        return False

    def beat(self) -> None:
        with self._lock:
            self._last = time.monotonic()

    def watch_event(self, event) -> None:
        """``event``: an object with ``query() -> bool`` (a recorded ``torch.cuda.Event``): the step's device work
        must complete within ``timeout_s`` of this call."""
        with self._lock:
            self._event = event
            self._event_since = time.monotonic()

    # ------------------------------------------------------------------- loop
    def _check(self) -> Optional[str]:
        now = time.monotonic()
        with self._lock:
            last, event, since = self._last, self._event, self._event_since
        if now - last > self.timeout_s:
            return f"no heartbeat for {now - last:.1f} s (limit {self.timeout_s:.1f} s)"
        if event is not None:
            try:
                done = bool(event.query())
            except Exception as e:  # noqa: BLE001 - a failed query is itself the finding
                return f"device event query failed: {e!r}"
            if done:
                with self._lock:
                    if self._event is event:
                        self._event = None
            elif now - since > self.timeout_s:
                return f"device work still pending after {now - since:.1f} s (limit {self.timeout_s:.1f} s)"
        if self.status_fn is not None:
            code = int(self.status_fn())
            if code != 0:
                return f"a kernel gave up on a bounded wait (status word {code})"
        return None

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            reason = self._check()
            if reason is not None:
                self.fired = reason
                self._stop.set()
                logger.error(f"watchdog: {reason}")
                try:
                    self.on_timeout(reason)
                except Exception:  # noqa: BLE001 - the watchdog thread must not die silently
                    logger.exception("watchdog callback failed")
                return

    @staticmethod
    def _interrupt_main(reason: str) -> None:
        import _thread

        faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        _thread.interrupt_main()
