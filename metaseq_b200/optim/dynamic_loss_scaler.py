"""Dynamic loss scale for fp16 training.

The schedule is the reference's non-standard one (metaseq/optim/dynamic_loss_scaler.py:11-75): after
``scale_window`` clean updates the scale doubles *and the window doubles too*; on overflow the scale halves
and the window halves (never below one update), subject to ``tolerance`` (fraction of updates since the last
rescale that may overflow before the scale is cut), ``threshold`` (floor applied when cutting) and
``min_loss_scale`` (the scale is never stored below it: the previous value is kept and the overflowing updates
keep being skipped).  An overflow is reported by raising ``OverflowError``.
"""
from __future__ import annotations

import math


class DynamicLossScaler:
    def __init__(self, init_scale=4.0, scale_factor=2.0, scale_window=256, tolerance=0.0, threshold=None,
                 min_loss_scale=2 ** -5):
        self.loss_scale = init_scale
        self.scale_factor = scale_factor
        self.scale_window = scale_window
        self.tolerance = tolerance
        self.threshold = threshold
        self.min_loss_scale = min_loss_scale
        # update counters: total, position of the last overflow / last rescale, overflows since that rescale
        self._iter = 0
        self._last_overflow_iter = -1
        self._last_rescale_iter = -1
        self._overflows_since_rescale = 0

    def scale(self, outputs):
        return outputs * self.loss_scale

    # ------------------------------------------------------------- clean update
    def update(self):
        """Bookkeeping after an update that did not overflow."""
        clean_run = self._iter - self._last_overflow_iter
        if clean_run % self.scale_window == 0:
            self._grow()
        self._iter += 1

    def _grow(self):
        self.loss_scale *= self.scale_factor
        self.scale_window *= self.scale_factor  # larger scales are probed less often
        self._last_rescale_iter = self._iter

    # ----------------------------------------------------------------- overflow
    def _decrease_loss_scale(self):
        cut = self.loss_scale / self.scale_factor
        self.loss_scale = cut if self.threshold is None else max(cut, self.threshold)
        self.scale_window = max(1, int(self.scale_window / self.scale_factor))

    def check_overflow(self, grad_norm):
        if not (math.isinf(grad_norm) or math.isnan(grad_norm)):
            return
        before = self.loss_scale
        since_rescale = max(1, self._iter - self._last_rescale_iter)
        self._last_overflow_iter = self._iter
        self._overflows_since_rescale += 1
        if self._overflows_since_rescale / since_rescale >= self.tolerance:
            self._decrease_loss_scale()
            self._last_rescale_iter = self._iter
            self._overflows_since_rescale = 0
        if self.loss_scale < self.min_loss_scale:
            self.loss_scale = before
        self._iter += 1
        raise OverflowError(f"setting loss scale to: {self.loss_scale}")
