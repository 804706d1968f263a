"""Batch iterators with resumable state.

``StreamingEpochBatchIterator`` drives an ``IterableDataset`` through a torch
``DataLoader`` and records, per DataLoader worker, how many sequences have been
consumed, so that a restart can fast-forward each worker independently
(reference: metaseq/data/iterators.py:210-418; state keys ``epoch``,
``sequences_consumed``, ``tokenization_cache``, ``n``, ``next_worker``).
``EpochBatchIterator`` is the map-style counterpart used by the legacy
language-modeling task and by inference (:421-685).  The small wrappers
(counting / grouped / sharded / buffered) follow :33-105 and :688-854.
"""
from __future__ import annotations

import itertools
import logging
import math
import os
import queue
import threading
import time
from typing import Callable, Iterable, List, Optional

import numpy as np
import torch

from metaseq_b200.data.document_to_sequence import DocumentToSequenceDataset

logger = logging.getLogger(__name__)

_SENTINEL = object()


class _Peekable:
    """Iterator with one element of look-ahead (``has_next``)."""

    def __init__(self, iterable):
        self._it = iter(iterable)
        self._head = _SENTINEL
        self._done = False

    def _fill(self):
        if self._head is _SENTINEL and not self._done:
            try:
                self._head = next(self._it)
            except StopIteration:
                self._done = True

    def has_next(self) -> bool:
        self._fill()
        return self._head is not _SENTINEL

    def __iter__(self):
        return self

    def __next__(self):
        self._fill()
        if self._head is _SENTINEL:
            raise StopIteration
        out, self._head = self._head, _SENTINEL
        return out


class CountingIterator:
    """Wraps an iterable and counts consumed elements (``n``); supports ``skip`` / ``take``."""

    def __init__(self, iterable, start: Optional[int] = None, total: Optional[int] = None):
        self.iterable = iterable
        self.itr = iter(self)
        self.n = start if start is not None else getattr(iterable, "n", 0)
        self.total = total if total is not None else self.n + len(iterable)

    def __len__(self):
        return self.total

    def __iter__(self):
        for x in self.iterable:
            if self.n >= self.total:
                raise RuntimeError("Mismatch between actual and expected iterable length.")
            self.n += 1
            yield x

    def __next__(self):
        return next(self.itr)

    def has_next(self) -> bool:
        return self.n < len(self)

    def skip(self, num_to_skip: int):
        next(itertools.islice(self.itr, num_to_skip, num_to_skip), None)
        return self

    def take(self, n: int):
        self.total = min(self.total, n)
        propagated = max(n - self.n, 0)
        if hasattr(self.iterable, "take"):
            self.iterable.take(propagated)
        else:
            self.iterable = itertools.islice(self.iterable, propagated)


class StreamingCountingIterator:
    """Counts batches and, per DataLoader worker, the sequences they stand for.  Each element
    of the wrapped iterable is ``(worker_id, batch)``."""

    def __init__(self, iterable, num_workers: int, batch_size: int, num_shards: int):
        self._itr = _Peekable(iterable)
        self.num_workers = max(1, num_workers)
        self.batch_size = batch_size
        self.num_shards = num_shards
        self.n = 0
        self.next_worker = 0
        self.sequences_consumed = [0] * self.num_workers
        self.worker_offset = 0

    def __iter__(self):
        return self

    def __next__(self):
        worker_id, batch = next(self._itr)
        worker_id = (worker_id + self.worker_offset) % self.num_workers
        self.sequences_consumed[worker_id] += self.batch_size * self.num_shards
        self.next_worker = (worker_id + 1) % self.num_workers
        self.n += 1
        return batch

    def __len__(self):
        return 0

    def has_next(self) -> bool:
        return self._itr.has_next()


def _abstract(name: str, doc: str):
    def method(self, *args, **kwargs):
        raise NotImplementedError(f"{type(self).__name__}.{name}")

    method.__name__, method.__doc__ = name, doc
    return method


class EpochBatchIterating:
    """What the trainer needs of an iterator that spans epochs."""

    __len__ = _abstract("__len__", "Batches per epoch.")
    next_epoch_itr = _abstract(
        "next_epoch_itr", "The iterator of the next epoch: (shuffle=True, fix_batches_to_gpus=False, "
        "set_dataset_epoch=True).")
    end_of_epoch = _abstract("end_of_epoch", "True once the current epoch's iterator is used up.")
    state_dict = _abstract("state_dict", "Position to resume from.")
    load_state_dict = _abstract("load_state_dict", "Moves to a saved position.")
    next_epoch_idx = property(_abstract("next_epoch_idx", "Number of the epoch that next_epoch_itr will start."))
    iterations_in_epoch = property(_abstract("iterations_in_epoch", "Batches consumed in the current epoch."))

    @property
    def first_batch(self):
        """A batch usable as a stand-in on ranks that run dry (or the string DUMMY when none can be made here)."""
        return "DUMMY"


class _TagWorker:
    def __init__(self, collate_fn):
        self.collate_fn = collate_fn

    def __call__(self, items):
        info = torch.utils.data.get_worker_info()
        return (info.id if info else 0, self.collate_fn(items))


def _find_doc_to_seq(dataset) -> DocumentToSequenceDataset:
    while not isinstance(dataset, DocumentToSequenceDataset):
        dataset = dataset.dataset
    return dataset


class StreamingEpochBatchIterator(EpochBatchIterating):
    def __init__(self, dataset, batch_size: int, collate_fn: Callable, drop_last: bool, num_workers: int = 0,
                 epoch: int = 1, num_shards: int = 1, pin_memory: bool = True):
        assert isinstance(dataset, torch.utils.data.IterableDataset)
        self.dataset = dataset
        self.batch_size = batch_size
        self.collate_fn = collate_fn
        self.drop_last = drop_last
        self.num_workers = num_workers
        self.epoch = max(epoch, 1)
        self.num_shards = num_shards
        self.pin_memory = pin_memory and torch.cuda.is_available()
        self._itr: Optional[StreamingCountingIterator] = None
        self.worker_offset = 0

    @property
    def next_epoch_idx(self):
        if self._itr is not None and self.end_of_epoch():
            return self.epoch + 1
        return self.epoch

    def next_epoch_itr(self, **kwargs):
        self.epoch = self.next_epoch_idx
        if self._itr is None or self.end_of_epoch():
            if hasattr(self.dataset, "set_epoch"):
                self.dataset.set_epoch(self.epoch)
            self._itr = self._make_iterator()
        return self._itr

    def end_of_epoch(self) -> bool:
        return not self._itr.has_next()

    @property
    def iterations_in_epoch(self) -> int:
        return self._itr.n

    def state_dict(self):
        from metaseq_b200.parallel import utils as dist_utils

        nw = max(1, self.num_workers)
        if self._itr is None or self.end_of_epoch():
            epoch = self.epoch + (0 if self._itr is None else 1)
            consumed, n, next_worker = [0] * nw, 0, 0
        else:
            epoch = self.epoch
            consumed, n, next_worker = list(self._itr.sequences_consumed), self._itr.n, self._itr.next_worker
        d2s = _find_doc_to_seq(self.dataset)
        return {
            "epoch": epoch,
            "sequences_consumed": consumed,
            "tokenization_cache": d2s.len_cache if dist_utils.get_global_rank() == 0 else None,
            "n": n,
            "next_worker": next_worker,
        }

    def load_state_dict(self, state_dict):
        from metaseq_b200.parallel import utils as dist_utils

        self.epoch = state_dict["epoch"]
        if hasattr(self.dataset, "set_epoch"):
            self.dataset.set_epoch(self.epoch)
        consumed = state_dict.get("sequences_consumed")
        if consumed and max(consumed) > 0:
            n, next_worker = state_dict["n"], state_dict["next_worker"]
            nw = max(1, self.num_workers)
            assert len(consumed) == nw, (
                "changing the number of workers in the middle of a shard changes the order the data will be loaded in"
            )
            per_batch = self.batch_size * self.num_shards
            if sum(consumed) != n * per_batch:
                logger.warning(f"sequences_consumed {consumed} does not add up to {n} x {per_batch}; rebuilding it")
                each, left = divmod(n, nw)
                consumed = [per_batch * (each + (1 if i < left else 0)) for i in range(nw)]
            d2s = _find_doc_to_seq(self.dataset)
            d2s.to_skip = list(consumed)
            d2s.worker_offset = next_worker
            self._restore_len_cache(d2s, state_dict.get("tokenization_cache"), dist_utils)
            self._itr = self._make_iterator()
            self._itr.n = n
            self._itr.sequences_consumed = list(consumed)
            self._itr.next_worker = next_worker
            self._itr.worker_offset = next_worker
        else:
            self._itr = self._make_iterator()
            pos = state_dict.get("iterations_in_epoch", 0)
            if pos > 0:
                logger.info(f"Fast-forwarding dataloader by {pos} batches (no tokenization cache in checkpoint)")
                next(itertools.islice(self._itr, pos, pos), None)

    @staticmethod
    def _restore_len_cache(d2s, cache, dist_utils):
        """Rank 0 owns the saved length cache; other ranks receive its bytes by broadcast."""
        group = dist_utils.get_global_group()
        if group is None or dist_utils.get_global_world_size() == 1:
            if cache is not None:
                d2s.len_cache = cache
                d2s.len_cache.set_num_workers(len(d2s.len_cache.worker_locks))
            return
        dev = dist_utils._comm_device(group)
        n_bytes = 4 * len(d2s.dataset)
        if dist_utils.get_global_rank() == 0 and cache is not None:
            d2s.len_cache = cache
            payload = torch.frombuffer(bytearray(cache.__getstate__()), dtype=torch.uint8).to(dev)
        else:
            payload = torch.zeros(n_bytes, dtype=torch.uint8, device=dev)
        dist_utils.broadcast(payload, 0, group)
        if dist_utils.get_global_rank() != 0:
            d2s.len_cache.load_bytes(payload.cpu().numpy().tobytes())

    def _make_iterator(self):
        if self.num_workers > 0:
            os.environ["PYTHONWARNINGS"] = "ignore:semaphore_tracker:UserWarning"
        d2s = None
        try:
            d2s = _find_doc_to_seq(self.dataset)
            d2s.set_num_workers(max(1, self.num_workers))
        except AttributeError:
            pass
        loader = torch.utils.data.DataLoader(
            dataset=self.dataset,
            batch_size=self.batch_size,
            num_workers=self.num_workers,
            collate_fn=_TagWorker(self.collate_fn),
            pin_memory=self.pin_memory,
            drop_last=self.drop_last,
            worker_init_fn=getattr(self.dataset, "worker_init_fn", None),
        )
        return StreamingCountingIterator(loader, self.num_workers, self.batch_size, self.num_shards)


class EpochBatchIterator(EpochBatchIterating):
    """Multi-epoch iterator over a map-style dataset with a precomputed batch sampler."""

    def __init__(self, dataset, collate_fn, batch_sampler, seed=1, num_shards=1, shard_id=0, num_workers=0, epoch=1,
                 buffer_size=0, timeout=0, disable_shuffling=False, skip_remainder_batch=True):
        assert isinstance(dataset, torch.utils.data.Dataset)
        self.dataset, self.collate_fn, self.batch_sampler = dataset, collate_fn, batch_sampler
        # a callable sampler is asked per epoch (lazily); a list of batches is fixed for good
        self._frozen_batches = None if callable(batch_sampler) else tuple(batch_sampler)
        self.seed, self.epoch = seed, max(epoch, 1)
        self.num_shards, self.shard_id = num_shards, shard_id
        self.num_workers, self.timeout = num_workers, timeout
        self.buffer_size = min(buffer_size, 20)  # more prefetched batches only cost memory
        self.disable_shuffling, self.shuffle = disable_shuffling, not disable_shuffling
        self.skip_remainder_batch = skip_remainder_batch
        self._supports_prefetch = getattr(dataset, "supports_prefetch", False)
        self._cur_epoch_itr = self._next_epoch_itr = None

    @property
    def frozen_batches(self):
        if self._frozen_batches is None:
            self._frozen_batches = tuple(self.batch_sampler(self.dataset, self.epoch))
        return self._frozen_batches

    @property
    def first_batch(self):
        if len(self.frozen_batches) == 0:
            raise Exception("The dataset is empty. This could indicate that all elements in the dataset have been "
                            "skipped. Try increasing the max number of allowed tokens or using a larger dataset.")
        if getattr(self.dataset, "supports_fetch_outside_dataloader", True):
            return self.collate_fn([self.dataset[i] for i in self.frozen_batches[0]])
        return "DUMMY"

    def __len__(self):
        return int(math.ceil(len(self.frozen_batches) / float(self.num_shards)))

    @property
    def n(self):
        return self.iterations_in_epoch

    @property
    def next_epoch_idx(self):
        if self._next_epoch_itr is not None:
            return self.epoch
        if self._cur_epoch_itr is not None and self.end_of_epoch():
            return self.epoch + 1
        return self.epoch

    def next_epoch_itr(self, shuffle=True, fix_batches_to_gpus=False, set_dataset_epoch=True):
        if self.disable_shuffling:
            shuffle = False
        self.epoch = self.next_epoch_idx
        if set_dataset_epoch and hasattr(self.dataset, "set_epoch"):
            self.dataset.set_epoch(self.epoch)
        if self._next_epoch_itr is not None:
            self._cur_epoch_itr, self._next_epoch_itr = self._next_epoch_itr, None
        else:
            if callable(self.batch_sampler):
                self._frozen_batches = None
            self._cur_epoch_itr = self._get_iterator_for_epoch(self.epoch, shuffle, fix_batches_to_gpus)
        self.shuffle = shuffle
        return self._cur_epoch_itr

    def end_of_epoch(self) -> bool:
        return not self._cur_epoch_itr.has_next()

    @property
    def iterations_in_epoch(self):
        if self._cur_epoch_itr is not None:
            return self._cur_epoch_itr.n
        if self._next_epoch_itr is not None:
            return self._next_epoch_itr.n
        return 0

    def state_dict(self):
        if self.end_of_epoch():
            epoch, pos = self.epoch + 1, 0
        else:
            epoch, pos = self.epoch, self.iterations_in_epoch
        return {"version": 2, "epoch": epoch, "iterations_in_epoch": pos, "shuffle": self.shuffle}

    def load_state_dict(self, state_dict):
        self.epoch = state_dict["epoch"]
        pos = state_dict.get("iterations_in_epoch", 0)
        version = state_dict.get("version", 1)
        if pos > 0:
            self._next_epoch_itr = self._get_iterator_for_epoch(self.epoch, shuffle=state_dict.get("shuffle", True),
                                                                offset=pos)
            if self._next_epoch_itr is None:
                if version == 1:
                    self.epoch += 1
                else:
                    raise RuntimeError("Cannot resume training due to dataloader mismatch; relaunch with "
                                       "--reset-dataloader")
        else:
            self._next_epoch_itr = None

    def _get_iterator_for_epoch(self, epoch, shuffle, fix_batches_to_gpus=False, offset=0):
        def shuffle_batches(batches, seed):
            from metaseq_b200.utils import numpy_seed

            with numpy_seed(seed):
                np.random.shuffle(batches)
            return batches

        if self._supports_prefetch:
            batches = list(self.frozen_batches)
            if shuffle and not fix_batches_to_gpus:
                batches = shuffle_batches(batches, self.seed + epoch)
            batches = list(ShardedIterator(batches, self.num_shards, self.shard_id, fill_value=[]))
            self.dataset.prefetch([i for s in batches for i in s])
            if shuffle and fix_batches_to_gpus:
                batches = shuffle_batches(batches, self.seed + epoch + self.shard_id)
        else:
            batches = list(self.frozen_batches)
            if shuffle:
                batches = shuffle_batches(batches, self.seed + epoch)
            batches = list(ShardedIterator(batches, self.num_shards, self.shard_id, fill_value=[]))
        if offset > 0 and offset >= len(batches):
            return None
        if self.num_workers > 0:
            os.environ["PYTHONWARNINGS"] = "ignore:semaphore_tracker:UserWarning"
        itr = torch.utils.data.DataLoader(self.dataset, collate_fn=self.collate_fn, batch_sampler=batches[offset:],
                                          num_workers=self.num_workers, timeout=self.timeout)
        if self.buffer_size > 0:
            itr = BufferedIterator(self.buffer_size, itr)
        itr = CountingIterator(itr, start=offset)
        if self.skip_remainder_batch:
            total = len(itr) - 1
            itr.take(total)
        return itr


class GroupedIterator(CountingIterator):
    """Yields lists of ``chunk_size`` consecutive elements (gradient accumulation groups)."""

    def __init__(self, iterable, chunk_size: int, skip_remainder_batch: bool = True):
        if skip_remainder_batch:
            total = int(math.floor(len(iterable) / float(chunk_size)))
        else:
            total = int(math.ceil(len(iterable) / float(chunk_size)))
        super().__init__(_chunks(iterable, chunk_size, skip_remainder_batch),
                         start=int(math.ceil(getattr(iterable, "n", 0) / float(chunk_size))), total=total)
        self.chunk_size = chunk_size

    def take(self, n):
        self.total = min(self.total, n)


def _chunks(iterable, chunk_size, skip_remainder_batch=False):
    chunk = []
    for x in iterable:
        chunk.append(x)
        if len(chunk) == chunk_size:
            yield chunk
            chunk = []
    if not skip_remainder_batch and chunk:
        yield chunk


class ShardedIterator(CountingIterator):
    """Every ``num_shards``-th element starting at ``shard_id``; short shards are filled."""

    def __init__(self, iterable, num_shards: int, shard_id: int, fill_value=None, skip_remainder_batch=None):
        if shard_id < 0 or shard_id >= num_shards:
            raise ValueError("shard_id must be between 0 and num_shards")
        n = len(iterable)
        sharded_len = n // num_shards if skip_remainder_batch else int(math.ceil(n / float(num_shards)))
        itr = map(
            lambda pair: pair[1],
            itertools.zip_longest(range(sharded_len), itertools.islice(iterable, shard_id, n, num_shards),
                                  fillvalue=fill_value),
        )
        super().__init__(itr, start=int(math.ceil(getattr(iterable, "n", 0) / float(num_shards))), total=sharded_len)


class BackgroundConsumer(threading.Thread):
    """Feeds a queue from an iterable on a daemon thread; the end of the stream is a sentinel, an error of the
    source is passed on as the exception object (metaseq/data/iterators.py:771-793)."""

    def __init__(self, q, source, max_len):
        super().__init__(daemon=True)
        self._queue, self._source, self._max_len = q, source, max_len
        self.count = 0

    def run(self):
        try:
            for item in self._source:
                self._queue.put(item)
                self.count += 1
                if self._max_len is not None and self.count >= self._max_len:
                    break
            self._queue.put(_SENTINEL)
        except Exception as e:  # surfaced to the consumer
            self._queue.put(e)


_BackgroundConsumer = BackgroundConsumer


class BufferedIterator:
    """Keeps up to ``size`` elements of ``iterable`` ready, produced by a background thread that starts with the
    first ``next``.  Complains (at debug level, at most every 15 minutes) when the buffer runs nearly empty after
    the first five minutes: a sign that data loading is the bottleneck."""

    _GRACE_S, _REPEAT_S = 5 * 60, 15 * 60

    def __init__(self, size: int, iterable):
        self._queue = queue.Queue(size)
        self._iterable, self.total = iterable, len(iterable)
        self._consumer = None
        self.start_time, self.warning_time = time.time(), None

    def __iter__(self):
        return self

    def __len__(self):
        return self.total

    def take(self, n):
        """Ends the stream after ``n`` elements (also told to the source, if it can do the same)."""
        self.total = min(self.total, n)
        inner = getattr(self._iterable, "take", None)
        if inner is not None:
            inner(n)
        return self

    def _note_starvation(self):
        now = time.time()
        low = self._queue.qsize() < min(2, max(1, self._queue.maxsize // 2))
        if low and now - self.start_time > self._GRACE_S and \
                (self.warning_time is None or now - self.warning_time > self._REPEAT_S):
            logger.debug("Data loading buffer is empty or nearly empty. This may indicate a data loading "
                         "bottleneck; increasing the number of workers (--num-workers) may help.")
            self.warning_time = now

    def __next__(self):
        if self._consumer is None:
            self._consumer = BackgroundConsumer(self._queue, self._iterable, self.total)
            self._consumer.start()
        self._note_starvation()
        item = self._queue.get(True)
        if item is _SENTINEL:
            raise StopIteration()
        if isinstance(item, Exception):
            raise item
        return item
