"""Dynamic loss scale for fp16 training.

The schedule is the reference's non-standard one (metaseq/optim/dynamic_loss_scaler.py:
11-75): after ``scale_window`` clean updates the scale doubles *and the window doubles
too*; on overflow the scale halves and the window halves (down to the initial window,
when one was given), subject to ``tolerance`` (fraction of recent updates allowed to
overflow), ``threshold`` (floor applied on decrease) and ``min_loss_scale`` (the scale
never drops below it; overflowing updates keep being skipped).
"""
from __future__ import annotations


class DynamicLossScaler:
    def __init__(self, init_scale=2.0 ** 15, scale_factor=2.0, scale_window=2000, tolerance=0.0, threshold=None,
                 min_loss_scale=1e-4):
        self.loss_scale = init_scale
        self.scale_factor = scale_factor
        self.scale_window = scale_window
        self.tolerance = tolerance
        self.threshold = threshold
        self.min_loss_scale = min_loss_scale
        self._iter = 0
        self._last_overflow_iter = -1
        self._last_rescale_iter = -1
        self._overflows_since_rescale = 0

    def scale(self, outputs):
        return self.loss_scale * outputs

    def update(self):
        """Call after every successful (non-overflow) update."""
        if (self._iter - self._last_overflow_iter) % self.scale_window == 0:
            self.loss_scale *= self.scale_factor
            self._last_rescale_iter = self._iter
            # the window grows with the scale so that very large scales are probed less often
            self.scale_window *= self.scale_factor
        self._iter += 1

    def _decrease_loss_scale(self):
        self.loss_scale /= self.scale_factor
        # halve the window as well, but never below 1 update
        self.scale_window = max(int(self.scale_window / self.scale_factor), 1)
        if self.threshold is not None:
            self.loss_scale = max(self.loss_scale, self.threshold)

    def check_overflow(self, grad_norm):
        if grad_norm == float("inf") or grad_norm != grad_norm:
            prev_scale = self.loss_scale
            iter_since_rescale = self._iter - self._last_rescale_iter
            self._last_overflow_iter = self._iter
            self._overflows_since_rescale += 1
            pct_overflow = self._overflows_since_rescale / float(max(iter_since_rescale, 1))
            if pct_overflow >= self.tolerance:
                self._decrease_loss_scale()
                self._last_rescale_iter = self._iter
                self._overflows_since_rescale = 0
            if self.loss_scale < self.min_loss_scale:
                # never go below the floor: keep the previous scale and keep skipping updates
                self.loss_scale = prev_scale
            self._iter += 1
            raise OverflowError("setting loss scale to: " + str(self.loss_scale))
