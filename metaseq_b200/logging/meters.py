"""Meters: running averages, sums, event rates and stopwatches with a serialisable state
(reference: metaseq/logging/meters.py).

Every meter declares the attributes that make up its checkpoint state in ``_STATE``; the base class turns that
into ``state_dict`` / ``load_state_dict`` and applies the optional rounding of the displayed value."""
from __future__ import annotations

import bisect
import time
from collections import OrderedDict
from typing import Dict, Optional

import torch


def _to_number(x):
    """Scalars leave the device when they are stored in a checkpoint."""
    if torch.is_tensor(x) and x.numel() == 1:
        return x.item()
    return x


def safe_round(number, ndigits):
    number = _to_number(number)
    return round(number, ndigits) if hasattr(number, "__round__") else number


class Meter:
    _STATE: tuple = ()

    def __init__(self, round: Optional[int] = None):
        self.round = round

    def reset(self):
        raise NotImplementedError

    def _raw_value(self):
        raise NotImplementedError

    @property
    def smoothed_value(self) -> float:
        value = self._raw_value()
        if value is None or self.round is None:
            return value
        return safe_round(value, self.round)

    def state_dict(self):
        state = {name: _to_number(getattr(self, name)) for name in self._STATE}
        if self._STATE:
            state["round"] = self.round
        return state

    def load_state_dict(self, state_dict):
        for name in self._STATE:
            setattr(self, name, state_dict[name])
        if self._STATE:
            self.round = state_dict.get("round", None)


class AverageMeter(Meter):
    """Weighted running average; ``val`` is the latest value."""

    _STATE = ("val", "sum", "count")

    def __init__(self, round: Optional[int] = None):
        super().__init__(round)
        self.reset()

    def reset(self):
        self.val, self.sum, self.count = None, 0, 0

    def update(self, val, n=1):
        if val is None:
            return
        self.val = val
        if n > 0:
            self.sum = self.sum + val * n
            self.count = self.count + n

    @property
    def avg(self):
        return self.val if self.count <= 0 else self.sum / self.count

    def _raw_value(self):
        return self.avg


class SumMeter(Meter):
    _STATE = ("sum",)

    def __init__(self, round: Optional[int] = None):
        super().__init__(round)
        self.reset()

    def reset(self):
        self.sum = 0

    def update(self, val):
        if val is not None:
            self.sum = self.sum + val

    def _raw_value(self):
        return self.sum


class TimeMeter(Meter):
    """Events per second since the meter was (re)started; ``init`` carries elapsed time across restarts."""

    def __init__(self, init: int = 0, n: int = 0, round: Optional[int] = None):
        super().__init__(round)
        self.reset(init, n)

    def reset(self, init=0, n=0):
        self.init, self.n, self.i = init, n, 0
        self.start = time.perf_counter()

    def update(self, val=1):
        self.n = self.n + val
        self.i += 1

    @property
    def elapsed_time(self):
        return self.init + (time.perf_counter() - self.start)

    @property
    def avg(self):
        return self.n / self.elapsed_time

    def _raw_value(self):
        return self.avg

    def state_dict(self):
        return {"init": self.elapsed_time, "n": _to_number(self.n), "round": self.round}

    def load_state_dict(self, state_dict):
        if "start" in state_dict:  # state written by very old checkpoints: only the elapsed time is usable
            self.reset(init=state_dict["init"])
            return
        self.reset(init=state_dict["init"], n=state_dict["n"])
        self.round = state_dict.get("round", None)


class StopwatchMeter(Meter):
    """Total / mean duration of an event bracketed by ``start`` and ``stop``."""

    _STATE = ("sum", "n")

    def __init__(self, round: Optional[int] = None):
        super().__init__(round)
        self.sum, self.n, self.start_time = 0, 0, None

    def start(self):
        self.start_time = time.perf_counter()

    def stop(self, n=1, prehook=None):
        if self.start_time is None:
            return
        if prehook is not None:
            prehook()  # typically a device synchronisation
        self.sum = self.sum + (time.perf_counter() - self.start_time)
        self.n = self.n + n

    def reset(self):
        self.sum, self.n = 0, 0
        self.start()

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        self.start_time = None

    @property
    def avg(self):
        return self.sum / self.n if self.n > 0 else self.sum

    @property
    def elapsed_time(self):
        return 0.0 if self.start_time is None else time.perf_counter() - self.start_time

    def _raw_value(self):
        return self.avg if self.sum > 0 else self.elapsed_time


class MetersDict(OrderedDict):
    """Meters kept in priority order (lower first, ties by insertion).  Derived meters hold a function of the
    whole dictionary and are evaluated on read; they are not checkpointed."""

    class _DerivedMeter(Meter):
        def __init__(self, fn):
            super().__init__()
            self.fn = fn

        def reset(self):
            pass

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.priorities = []

    def __setitem__(self, key, value):
        assert key not in self, "MetersDict doesn't support reassignment"
        priority, meter = value
        bisect.insort(self.priorities, (priority, len(self.priorities), key))
        super().__setitem__(key, meter)
        for _, _, name in self.priorities:  # restore priority order after the append
            self.move_to_end(name)

    def add_meter(self, key, meter, priority):
        self[key] = (priority, meter)

    def _is_derived(self, key) -> bool:
        return isinstance(self[key], MetersDict._DerivedMeter)

    def get_smoothed_value(self, key: str) -> float:
        meter = self[key]
        return meter.fn(self) if self._is_derived(key) else meter.smoothed_value

    def get_smoothed_values(self) -> Dict[str, float]:
        return OrderedDict((k, self.get_smoothed_value(k)) for k in self if not k.startswith("_"))

    def reset(self):
        for key, meter in self.items():
            if not self._is_derived(key):
                meter.reset()

    def state_dict(self):
        return [(pri, key, type(self[key]).__name__, self[key].state_dict())
                for pri, _, key in self.priorities if not self._is_derived(key)]

    def load_state_dict(self, state_dict):
        self.clear()
        self.priorities.clear()
        for pri, key, cls_name, meter_state in state_dict:
            meter = globals()[cls_name]()
            meter.load_state_dict(meter_state)
            self.add_meter(key, meter, pri)
