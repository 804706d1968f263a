"""Per-module slots inside the ``incremental_state`` dictionary used during step-by-step decoding.

Each module instance gets a unique number at construction; its entries live under ``<number>.<key>`` so several
instances of the same class can share one dictionary (reference: metaseq/incremental_decoding_utils.py:13-69).
The attention module here keeps its preallocated key/value cache under such a key."""
from __future__ import annotations

import itertools
from typing import Dict, Optional, Protocol, runtime_checkable

from torch import Tensor


Slot = Dict[str, Optional[Tensor]]   # one module's entries
Slots = Dict[str, Slot]              # the dictionary shared by all modules of a decoder


@runtime_checkable
class HasIncrementalState(Protocol):
    """What ``with_incremental_state`` gives a module: access to its own slot of the shared dictionary."""

    def get_incremental_state(self, incremental_state: Optional[Slots], key: str) -> Optional[Slot]: ...

    def set_incremental_state(self, incremental_state: Optional[Slots], key: str, value: Slot) -> Optional[Slots]: ...


_instance_numbers = itertools.count()


class IncrementalState:
    """Mixin: every instance draws a process-wide number at construction and files its entries under
    ``"<number>.<key>"``, so any number of modules can share one dictionary without colliding."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.init_incremental_state()

    def init_incremental_state(self) -> None:
        self._slot_prefix = f"{next(_instance_numbers)}."

    def get_incremental_state(self, incremental_state: Optional[Slots], key: str) -> Optional[Slot]:
        return None if incremental_state is None else incremental_state.get(self._slot_prefix + key)

    def set_incremental_state(self, incremental_state: Optional[Slots], key: str, value: Slot) -> Optional[Slots]:
        if incremental_state is not None:
            incremental_state[self._slot_prefix + key] = value
        return incremental_state


def with_incremental_state(cls):
    """Class decorator: mixes ``IncrementalState`` into ``cls`` (ahead of its other bases)."""
    cls.__bases__ = (IncrementalState,) + tuple(b for b in cls.__bases__ if b is not IncrementalState)
    return cls
