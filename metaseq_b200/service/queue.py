"""Priority queues sharded by a key, so that requests with the same generation settings can be
batched together: ``get_largest_queue`` picks the fullest shard (reference:
metaseq/service/queue.py:11-108)."""
from __future__ import annotations

import hashlib
import queue
import random
import threading
from collections import defaultdict


class KeyedPriorityQueueCollection:
    """One ``PriorityQueue`` per key, created on first ``put``."""

    def __init__(self):
        self.queues = {}
        self._lock = threading.Lock()

    def put(self, key, item):
        with self._lock:
            q = self.queues.get(key)
            if q is None:
                q = self.queues[key] = queue.PriorityQueue()
        q.put(item)

    def get_largest_queue_key(self):
        with self._lock:
            if not self.queues:
                return None
            return max(self.queues, key=lambda k: self.queues[k].qsize())

    def get_largest_queue(self):
        key = self.get_largest_queue_key()
        return self.queues[key] if key is not None else None


class PriorityQueueRingShardKeyable:
    def queue_key(self):
        raise NotImplementedError


class PriorityQueueRingShard:
    """A group of keyed queues that tracks its total size (the deepest queue drives batching)."""

    @staticmethod
    def key_from_dict(d: dict) -> str:
        return ":".join(f"{k}={d[k]}" for k in sorted(d))

    @staticmethod
    def key_from_dictionary(key_dict: dict) -> str:
        """The reference's spelling of a shard key: ``k1:v1:k2:v2`` over the sorted keys."""
        return ":".join(f"{k}:{key_dict[k]}" for k in sorted(key_dict))

    @staticmethod
    def get_shard_index_for_key(key: str, num_shards: int = 1, deskew_factor: int = 1) -> int:
        """SHA-1 of the key modulo the number of shards: the same in every process, unlike ``hash``.  A
        ``deskew_factor`` > 1 spreads a hot key over shards by a random prefix (then it is not deterministic)."""
        if deskew_factor > 1:
            key = f"{random.randint(0, deskew_factor * num_shards)}:{key}"
        return int(hashlib.sha1(key.encode("utf-8")).hexdigest(), 16) % num_shards

    def __init__(self):
        self.queues = defaultdict(queue.PriorityQueue)
        self.deepest_queue_key = None
        self.size = 0
        self._lock = threading.Lock()

    def put(self, key, item):
        with self._lock:
            q = self.queues[key]
            q.put(item)
            self.size += 1
            if self.deepest_queue_key is None or q.qsize() > self.queues[self.deepest_queue_key].qsize():
                self.deepest_queue_key = key

    def _recompute_deepest(self):
        self.deepest_queue_key = max(self.queues, key=lambda k: self.queues[k].qsize()) if self.queues else None

    def get_deepest_queue(self):
        with self._lock:
            if self.deepest_queue_key is None:
                return None
            return self.queues[self.deepest_queue_key]

    def get(self, key=None, block=False, timeout=None):
        with self._lock:
            if key is None:
                key = self.deepest_queue_key
            if key is None:
                raise queue.Empty
            q = self.queues[key]
        item = q.get(block=block, timeout=timeout)
        with self._lock:
            self.size -= 1
            self._recompute_deepest()
        return item

    def empty(self):
        return self.size == 0


class PriorityQueueRing:
    """Several shards; producers hash to a shard, the consumer drains the largest shard."""

    def __init__(self, num_shards: int = 1, deskew_factor: int = 1):
        self.shards = [PriorityQueueRingShard() for _ in range(num_shards)]
        self.deskew_factor = deskew_factor

    def put(self, item: PriorityQueueRingShardKeyable):
        key = item.queue_key()
        index = PriorityQueueRingShard.get_shard_index_for_key(key, len(self.shards), self.deskew_factor)
        self.shards[index].put(key, item)

    def largest_shard(self):
        return max(self.shards, key=lambda s: s.size)

    def empty(self):
        return all(s.empty() for s in self.shards)
