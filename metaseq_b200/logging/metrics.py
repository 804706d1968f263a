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
from collections import defaultdict
from typing import Callable, Dict, List, Optional

from .meters import AverageMeter, Meter, MetersDict, StopwatchMeter, SumMeter, TimeMeter

logger = logging.getLogger(__name__)

_aggregators = {}
_active_aggregators = {}
_active_aggregators_cnt = defaultdict(lambda: 0)


def reset() -> None:
    _aggregators.clear()
    _active_aggregators.clear()
    _active_aggregators_cnt.clear()
    _aggregators["default"] = MetersDict()
    _active_aggregators["default"] = _aggregators["default"]
    _active_aggregators_cnt["default"] = 1


reset()


@contextlib.contextmanager
def aggregate(name: Optional[str] = None, new_root: bool = False):
    if name is None:
        name = str(uuid.uuid4())
        assert name not in _aggregators
        agg = MetersDict()
    else:
        assert name != "default"
        agg = _aggregators.setdefault(name, MetersDict())
    if new_root:
        backup = _active_aggregators.copy()
        _active_aggregators.clear()
        backup_cnt = _active_aggregators_cnt.copy()
        _active_aggregators_cnt.clear()
    _active_aggregators[name] = agg
    _active_aggregators_cnt[name] += 1
    yield agg
    _active_aggregators_cnt[name] -= 1
    if _active_aggregators_cnt[name] == 0 and name in _active_aggregators:
        del _active_aggregators[name]
    if new_root:
        _active_aggregators.clear()
        _active_aggregators.update(backup)
        _active_aggregators_cnt.clear()
        _active_aggregators_cnt.update(backup_cnt)


def get_active_aggregators() -> List[MetersDict]:
    return list(_active_aggregators.values())


def log_scalar(key: str, value: float, weight: float = 1, priority: int = 10, round: Optional[int] = None):
    for agg in get_active_aggregators():
        if key not in agg:
            agg.add_meter(key, AverageMeter(round=round), priority)
        agg[key].update(value, weight)


def log_scalar_sum(key: str, value: float, priority: int = 10, round: Optional[int] = None):
    for agg in get_active_aggregators():
        if key not in agg:
            agg.add_meter(key, SumMeter(round=round), priority)
        agg[key].update(value)


def log_derived(key: str, fn: Callable[[MetersDict], float], priority: int = 20):
    for agg in get_active_aggregators():
        if key not in agg:
            agg.add_meter(key, MetersDict._DerivedMeter(fn), priority)


def log_speed(key: str, value: float, priority: int = 30, round: Optional[int] = None):
    for agg in get_active_aggregators():
        if key not in agg:
            agg.add_meter(key, TimeMeter(round=round), priority)
            agg[key].reset()
        else:
            agg[key].update(value)


def log_start_time(key: str, priority: int = 40, round: Optional[int] = None):
    for agg in get_active_aggregators():
        if key not in agg:
            agg.add_meter(key, StopwatchMeter(round=round), priority)
        agg[key].start()


def log_stop_time(key: str, weight: float = 0.0, prehook=None):
    for agg in get_active_aggregators():
        if key in agg:
            agg[key].stop(weight, prehook)


def log_custom(new_meter_fn: Callable[[], Meter], key: str, *args, priority: int = 50, **kwargs):
    for agg in get_active_aggregators():
        if key not in agg:
            agg.add_meter(key, new_meter_fn(), priority)
        agg[key].update(*args, **kwargs)


def reset_meter(name: str, key: str) -> None:
    meter = get_meter(name, key)
    if meter is not None:
        meter.reset()


def reset_meters(name: str) -> None:
    meters = get_meters(name)
    if meters is not None:
        meters.reset()


def get_meter(name: str, key: str) -> Meter:
    if name not in _aggregators:
        return None
    return _aggregators[name].get(key, None)


def get_meters(name: str) -> MetersDict:
    return _aggregators.get(name, None)


def get_smoothed_value(name: str, key: str) -> float:
    return _aggregators[name].get_smoothed_value(key)


def get_smoothed_values(name: str) -> Dict[str, float]:
    return _aggregators[name].get_smoothed_values()


def state_dict():
    return {name: agg.state_dict() for name, agg in _aggregators.items()}


def load_state_dict(state_dict):
    for name, agg_state in state_dict.items():
        _aggregators[name] = MetersDict()
        _aggregators[name].load_state_dict(agg_state)


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
