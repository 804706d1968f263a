"""Extra rendezvous schemes for ``init_process_group``: ``tcpr://host:port`` retries the TCP
store connection with exponential backoff (flaky cluster start-up), ``barrierlesstcpr://`` also
skips the store-based barrier at the end of initialisation (reference:
metaseq/distributed/rendezvous.py:39-131)."""
from __future__ import annotations

import logging
import random
import time
from datetime import timedelta
from urllib.parse import urlparse

import torch.distributed as dist
from torch.distributed.rendezvous import register_rendezvous_handler

logger = logging.getLogger(__name__)
_MAX_RETRIES = 5


def _query(url):
    q = dict(pair.split("=") for pair in filter(None, url.query.split("&")))
    if "rank" not in q or "world_size" not in q:
        raise ValueError(f"tcpr rendezvous needs rank and world_size in the URL: {url.geturl()}")
    return int(q["rank"]), int(q["world_size"])


def _store_with_retries(host, port, rank, world_size, timeout):
    delay = 1.0
    for attempt in range(_MAX_RETRIES):
        try:
            return dist.TCPStore(host, port, world_size, rank == 0, timeout, multi_tenant=True)
        except RuntimeError as e:
            if attempt == _MAX_RETRIES - 1:
                raise
            logger.warning(f"TCPStore connection failed ({e}); retry {attempt + 1}/{_MAX_RETRIES} in {delay:.1f}s")
            time.sleep(delay + random.random())
            delay *= 2


class _BarrierlessStore(dist.Store):
    """Delegates to a TCP store but answers the init barrier's counter keys locally, so no rank
    waits on the others at the end of ``init_process_group``."""

    def __init__(self, inner, world_size):
        super().__init__()
        self.inner = inner
        self.world_size = world_size

    def set(self, k, v):
        return self.inner.set(k, v)

    def get(self, k):
        return self.inner.get(k)

    def add(self, k, n):
        if "store_based_barrier_key" in k:
            return self.world_size
        return self.inner.add(k, n)

    def wait(self, keys, timeout=None):
        return self.inner.wait(keys) if timeout is None else self.inner.wait(keys, timeout)

    def set_timeout(self, t):
        return self.inner.set_timeout(t)

    def num_keys(self):
        return self.inner.num_keys()

    def delete_key(self, k):
        return self.inner.delete_key(k)


ComplicitStore = _BarrierlessStore  # the reference's name for it (metaseq/distributed/rendezvous.py)


def _tcpr_handler(url, timeout=timedelta(minutes=30), **kwargs):
    u = urlparse(url)
    rank, world_size = _query(u)
    store = _store_with_retries(u.hostname, u.port, rank, world_size, timeout)
    yield (store, rank, world_size)
    raise RuntimeError("Unable to perform re-rendezvous using tcpr:// method")


def _barrierless_handler(url, timeout=timedelta(minutes=30), **kwargs):
    u = urlparse(url)
    rank, world_size = _query(u)
    store = _BarrierlessStore(_store_with_retries(u.hostname, u.port, rank, world_size, timeout), world_size)
    yield (store, rank, world_size)
    raise RuntimeError("Unable to perform re-rendezvous using barrierlesstcpr:// method")


def register():
    for scheme, handler in (("tcpr", _tcpr_handler), ("barrierlesstcpr", _barrierless_handler)):
        try:
            register_rendezvous_handler(scheme, handler)
        except RuntimeError:
            pass  # already registered


register()
