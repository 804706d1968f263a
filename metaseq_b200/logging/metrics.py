"""Named, nestable metric aggregators.

``with metrics.aggregate("train"):`` opens an aggregation context; every
``log_scalar`` / ``log_speed`` / ``log_derived`` call inside feeds all active contexts
(and the always-on ``default`` one).  Reference: metaseq/logging/metrics.py:52-209,
state dict :288-295, nvidia-smi parsing :298-329.
"""
from __future__ import annotations

import contextlib
import logging
import subprocess
import uuid
from typing import Callable, Dict, List, Optional

from .meters import AverageMeter, Meter, MetersDict, StopwatchMeter, SumMeter, TimeMeter

logger = logging.getLogger(__name__)

class AggregatorStack:
    """All named aggregators of the process plus the set that currently receives log calls.

    ``named`` maps a name to its ``MetersDict`` and lives until ``reset``; ``live`` maps the name of every open
    scope (and ``default``, which is always open) to ``[meters, depth]`` so that a scope entered twice under the
    same name closes only with its outermost exit."""

    def __init__(self):
        self.named: Dict[str, MetersDict] = {}
        self.live: Dict[str, list] = {}
        self.reset()

    def reset(self):
        self.named.clear()
        self.live.clear()
        self.named["default"] = MetersDict()
        self.live["default"] = [self.named["default"], 1]

    def open(self, name: Optional[str], new_root: bool):
        """Enters a scope; returns ``(key, meters, saved)`` where ``saved`` is the suspended live set of a new root."""
        if name == "default":
            raise ValueError("the default aggregator is always open")
        if name is None:  # an anonymous scope is not kept after it closes
            key, meters = "anonymous-" + uuid.uuid4().hex, MetersDict()
        else:
            key, meters = name, self.named.setdefault(name, MetersDict())
        saved = None
        if new_root:
            saved, self.live = self.live, {}
        entry = self.live.setdefault(key, [meters, 0])
        entry[1] += 1
        return key, meters, saved

    def close(self, key: str, saved):
        entry = self.live.get(key)
        if entry is not None:
            entry[1] -= 1
            if entry[1] <= 0:
                del self.live[key]
        if saved is not None:
            self.live = saved

    def receivers(self) -> List[MetersDict]:
        return [entry[0] for entry in self.live.values()]

    def feed(self, key: str, factory: Callable[[], Meter], priority: int, update: Optional[Callable[[Meter, bool], None]]):
        """Makes sure every receiving aggregator has a meter ``key`` (built by ``factory``) and applies
        ``update(meter, created_now)`` to it."""
        for meters in self.receivers():
            created = key not in meters
            if created:
                meters.add_meter(key, factory(), priority)
            if update is not None:
                update(meters[key], created)


_STACK = AggregatorStack()


def reset() -> None:
    _STACK.reset()


class aggregate(contextlib.ContextDecorator):
    """``with aggregate("train") as meters:`` or ``@aggregate("train")``: log calls made inside also feed the
    aggregator of that name (a throw-away one without a name).  ``new_root`` suspends the enclosing scopes, the
    default one included, for the duration."""

    def __init__(self, name: Optional[str] = None, new_root: bool = False):
        self.name, self.new_root = name, new_root
        self._entered = []

    def _recreate_cm(self):  # a decorated function may recurse: every call gets its own scope object
        return aggregate(self.name, self.new_root)

    def __enter__(self) -> MetersDict:
        key, meters, saved = _STACK.open(self.name, self.new_root)
        self._entered.append((key, saved))
        return meters

    def __exit__(self, *exc):
        key, saved = self._entered.pop()
        _STACK.close(key, saved)
        return False


def get_active_aggregators() -> List[MetersDict]:
    return _STACK.receivers()


def log_scalar(key: str, value: float, weight: float = 1, priority: int = 10, round: Optional[int] = None):
    """Weighted running average of ``value``."""
    _STACK.feed(key, lambda: AverageMeter(round=round), priority, lambda m, _new: m.update(value, weight))


def log_scalar_sum(key: str, value: float, priority: int = 10, round: Optional[int] = None):
    """Running sum of ``value``."""
    _STACK.feed(key, lambda: SumMeter(round=round), priority, lambda m, _new: m.update(value))


def log_derived(key: str, fn: Callable[[MetersDict], float], priority: int = 20):
    """A value computed from the other meters of the aggregator when it is read."""
    _STACK.feed(key, lambda: MetersDict._DerivedMeter(fn), priority, None)


def log_speed(key: str, value: float, priority: int = 30, round: Optional[int] = None):
    """``value`` per second; the clock starts with the first call, which itself counts nothing."""
    _STACK.feed(key, lambda: TimeMeter(round=round), priority,
                lambda m, new: m.reset() if new else m.update(value))


def log_start_time(key: str, priority: int = 40, round: Optional[int] = None):
    _STACK.feed(key, lambda: StopwatchMeter(round=round), priority, lambda m, _new: m.start())


def log_stop_time(key: str, weight: float = 0.0, prehook=None):
    for meters in _STACK.receivers():
        if key in meters:
            meters[key].stop(weight, prehook)


def log_custom(new_meter_fn: Callable[[], Meter], key: str, *args, priority: int = 50, **kwargs):
    _STACK.feed(key, new_meter_fn, priority, lambda m, _new: m.update(*args, **kwargs))


def get_meters(name: str) -> Optional[MetersDict]:
    return _STACK.named.get(name)


def get_meter(name: str, key: str) -> Optional[Meter]:
    meters = get_meters(name)
    return None if meters is None else meters.get(key)


def reset_meters(name: str) -> None:
    meters = get_meters(name)
    if meters is not None:
        meters.reset()


def reset_meter(name: str, key: str) -> None:
    meter = get_meter(name, key)
    if meter is not None:
        meter.reset()


def get_smoothed_value(name: str, key: str) -> float:
    return _STACK.named[name].get_smoothed_value(key)


def get_smoothed_values(name: str) -> Dict[str, float]:
    return _STACK.named[name].get_smoothed_values()


def state_dict():
    return {name: meters.state_dict() for name, meters in _STACK.named.items()}


def load_state_dict(state_dict):
    """Replaces the named aggregators with the saved ones; open scopes keep feeding the restored objects."""
    for name, saved in state_dict.items():
        meters = MetersDict()
        meters.load_state_dict(saved)
        _STACK.named[name] = meters
        if name in _STACK.live:
            _STACK.live[name][0] = meters


def nvidia_smi_gpu_memory_stats():
    """``{gpu_<i>_mem_used_gb: float}`` parsed from ``nvidia-smi --query-gpu=memory.used``."""
    out = {}
    try:
        text = subprocess.check_output(
            ["nvidia-smi", "--query-gpu=index,memory.used", "--format=csv,noheader,nounits"], timeout=10
        ).decode("utf-8")
        for line in text.strip().splitlines():
            idx, used = [s.strip() for s in line.split(",")]
            out[f"gpu_{idx}_mem_used_gb"] = float(used) / 1024.0
    except Exception as e:  # nvidia-smi missing or unresponsive
        logger.debug(f"nvidia-smi query failed: {e}")
    return out


def get_nvidia_smi_gpu_memory_stats_str():
    return "nvidia-smi stats: {}".format(nvidia_smi_gpu_memory_stats())
