"""Per-module slots inside the ``incremental_state`` dictionary used during step-by-step decoding.

Each module instance gets a unique id at construction; its entries live under ``<id>.<key>`` so several
instances of the same class can share one dictionary (reference: metaseq/incremental_decoding_utils.py:13-69).
The attention module here keeps its preallocated key/value cache under such a key."""
from __future__ import annotations

import uuid
from typing import Dict, Optional, Protocol, runtime_checkable

from torch import Tensor


@runtime_checkable
class HasIncrementalState(Protocol):
    """What ``with_incremental_state`` gives a module: typed access to its own slot of the shared dictionary."""

    def get_incremental_state(self, incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]],
                              key: str) -> Optional[Dict[str, Optional[Tensor]]]:
        ...

    def set_incremental_state(self, incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]], key: str,
                              value: Dict[str, Optional[Tensor]]) -> Optional[Dict[str, Dict[str, Optional[Tensor]]]]:
        ...


class IncrementalState:
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.init_incremental_state()

    def init_incremental_state(self):
        self._incremental_state_id = str(uuid.uuid4())

    def _get_full_incremental_state_key(self, key: str) -> str:
        return f"{self._incremental_state_id}.{key}"

    def get_incremental_state(self, incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]],
                              key: str) -> Optional[Dict[str, Optional[Tensor]]]:
        if incremental_state is None:
            return None
        return incremental_state.get(self._get_full_incremental_state_key(key))

    def set_incremental_state(self, incremental_state: Optional[Dict[str, Dict[str, Optional[Tensor]]]], key: str,
                              value: Dict[str, Optional[Tensor]]):
        if incremental_state is not None:
            incremental_state[self._get_full_incremental_state_key(key)] = value
        return incremental_state


def with_incremental_state(cls):
    """Class decorator: mixes ``IncrementalState`` into ``cls`` (ahead of its other bases)."""
    cls.__bases__ = (IncrementalState,) + tuple(b for b in cls.__bases__ if b is not IncrementalState)
    return cls
