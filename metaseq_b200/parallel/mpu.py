"""Process-group layout for data x tensor parallelism and the per-group RNG tracker.

Rank layout is the reference's (metaseq/modules/megatron/mpu/initialize.py:124-161):
tensor-parallel ranks are contiguous ``[i*tp, (i+1)*tp)``; data-parallel ranks are
strided by ``tp``.  There is no pipeline parallelism.  The RNG tracker reproduces
metaseq/modules/megatron/mpu/random.py:178-220: the default generator is seeded
with ``seed`` on every rank, a separate "model-parallel" stream with
``seed + 2718 + tp_rank`` is forked around dropout inside tensor-parallel regions.
"""
from __future__ import annotations

import contextlib
from typing import Dict, Optional

import torch
import torch.distributed as dist

_TP_GROUP = None
_DP_GROUP = None
_MP_GROUP = None  # equals the TP group (no pipeline stage dimension)
_TP_RANKS = None
_DP_RANKS = None
_TP_SIZE = 1
_INITIALIZED = False


def initialize_model_parallel(tensor_model_parallel_size: int = 1, backend: Optional[str] = None) -> None:
    global _TP_GROUP, _DP_GROUP, _MP_GROUP, _TP_RANKS, _DP_RANKS, _TP_SIZE, _INITIALIZED
    assert dist.is_initialized()
    world = dist.get_world_size()
    rank = dist.get_rank()
    tp = min(int(tensor_model_parallel_size), world)
    if world % tp != 0:
        raise RuntimeError(f"world size {world} is not divisible by tensor parallel size {tp}")
    dp = world // tp
    # every rank must create every group, in the same order
    for j in range(tp):
        ranks = list(range(j, world, tp))
        g = dist.new_group(ranks, backend=backend)
        if rank in ranks:
            _DP_GROUP, _DP_RANKS = g, ranks
    for i in range(dp):
        ranks = list(range(i * tp, (i + 1) * tp))
        g = dist.new_group(ranks, backend=backend)
        if rank in ranks:
            _TP_GROUP, _TP_RANKS = g, ranks
    _MP_GROUP = _TP_GROUP
    _TP_SIZE = tp
    _INITIALIZED = True


def model_parallel_is_initialized() -> bool:
    return _INITIALIZED


def destroy_model_parallel():
    global _TP_GROUP, _DP_GROUP, _MP_GROUP, _TP_RANKS, _DP_RANKS, _TP_SIZE, _INITIALIZED
    _TP_GROUP = _DP_GROUP = _MP_GROUP = _TP_RANKS = _DP_RANKS = None
    _TP_SIZE = 1
    _INITIALIZED = False


def get_tensor_model_parallel_group():
    return _TP_GROUP


def get_model_parallel_group():
    return _MP_GROUP


def get_data_parallel_group():
    return _DP_GROUP


def get_tensor_model_parallel_world_size() -> int:
    return _TP_SIZE if _INITIALIZED else 1


def get_tensor_model_parallel_rank() -> int:
    if not _INITIALIZED or _TP_SIZE == 1:
        return 0
    return dist.get_rank(group=_TP_GROUP)


def get_tensor_model_parallel_ranks():
    return _TP_RANKS or [dist.get_rank() if dist.is_initialized() else 0]


def get_data_parallel_ranks():
    return _DP_RANKS or [dist.get_rank() if dist.is_initialized() else 0]


def get_tensor_model_parallel_src_rank() -> int:
    g = dist.get_rank() if dist.is_initialized() else 0
    return (g // max(1, _TP_SIZE)) * max(1, _TP_SIZE)


def get_data_parallel_world_size() -> int:
    if not _INITIALIZED:
        return dist.get_world_size() if dist.is_initialized() else 1
    return dist.get_world_size(group=_DP_GROUP)


def get_data_parallel_rank() -> int:
    if not _INITIALIZED:
        return dist.get_rank() if dist.is_initialized() else 0
    return dist.get_rank(group=_DP_GROUP)


def ensure_divisibility(a: int, b: int) -> None:
    assert a % b == 0, f"{a} is not divisible by {b}"


def divide(a: int, b: int) -> int:
    ensure_divisibility(a, b)
    return a // b


def vocab_range(global_vocab: int, rank: int, world: int):
    per = divide(global_vocab, world)
    return rank * per, (rank + 1) * per


class VocabUtility:
    """[first, last) of the vocabulary rows that ``rank`` owns (reference:
    metaseq/modules/megatron/mpu/utils.py:47-63)."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition_vocab_size: int, rank: int):
        return rank * per_partition_vocab_size, (rank + 1) * per_partition_vocab_size

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab_size: int, rank: int, world_size: int):
        return vocab_range(global_vocab_size, rank, world_size)


def split_tensor_along_last_dim(tensor: torch.Tensor, num_partitions: int, contiguous_split_chunks: bool = False):
    """``num_partitions`` equal views of the last dimension (copies if ``contiguous_split_chunks``)."""
    pieces = torch.split(tensor, divide(tensor.size(-1), num_partitions), dim=-1)
    return tuple(p.contiguous() for p in pieces) if contiguous_split_chunks else pieces


_PARTITION_ATTRIBUTES = {"tensor_model_parallel": False, "partition_dim": -1, "partition_stride": 1}


def set_tensor_model_parallel_attributes(tensor, is_parallel: bool, dim: int, stride: int = 1) -> None:
    """Marks a parameter as one rank's slice of a larger tensor: checkpoint tools and gradient-norm code read
    ``tensor_model_parallel`` / ``partition_dim`` / ``partition_stride`` (reference:
    metaseq/modules/megatron/mpu/layers.py:34-47); ``model_parallel`` is the flag that the trainer's
    gradient-norm reduction looks at."""
    for name in _PARTITION_ATTRIBUTES:
        assert not hasattr(tensor, name), f"{name} is already set"
    tensor.tensor_model_parallel = is_parallel
    tensor.partition_dim = dim
    tensor.partition_stride = stride
    tensor.model_parallel = is_parallel


def param_is_tensor_parallel(param) -> bool:
    return bool(getattr(param, "tensor_model_parallel", False))


# ------------------------------------------------------------------- RNG
_MODEL_PARALLEL_RNG = "model-parallel-rng"


class RNGStatesTracker:
    """Named RNG states that can be forked into and restored from.  Works on CPU (torch
    default generator) and CUDA (the current device's generator)."""

    def __init__(self):
        self.states_: Dict[str, torch.Tensor] = {}
        self.seeds_ = set()

    def reset(self):
        self.states_ = {}
        self.seeds_ = set()

    def get_states(self):
        return {k: v.clone() for k, v in self.states_.items()}

    def set_states(self, states):
        self.states_ = {k: v.clone() for k, v in states.items()}

    @staticmethod
    def _get():
        return torch.cuda.get_rng_state() if torch.cuda.is_available() else torch.get_rng_state()

    @staticmethod
    def _set(state):
        if torch.cuda.is_available():
            torch.cuda.set_rng_state(state)
        else:
            torch.set_rng_state(state)

    def add(self, name: str, seed: int):
        if seed in self.seeds_:
            raise Exception(f"seed {seed} already exists")
        if name in self.states_:
            raise Exception(f"rng state {name} already exists")
        self.seeds_.add(seed)
        orig = self._get()
        if torch.cuda.is_available():
            torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states_[name] = self._get()
        self._set(orig)

    @contextlib.contextmanager
    def fork(self, name: str = _MODEL_PARALLEL_RNG):
        if name not in self.states_:
            yield
            return
        orig = self._get()
        self._set(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = self._get()
            self._set(orig)


_RNG_TRACKER = RNGStatesTracker()


CudaRNGStatesTracker = RNGStatesTracker  # the reference's name (metaseq/modules/megatron/mpu/random.py:98)


def get_cuda_rng_tracker() -> RNGStatesTracker:
    return _RNG_TRACKER


def model_parallel_cuda_manual_seed(seed: int):
    """Default stream: ``seed`` on all ranks (identical dropout in replicated regions);
    model-parallel stream: ``seed + 2718 + tp_rank`` (different dropout per partition)."""
    tp_seed = seed + 2718 + get_tensor_model_parallel_rank()
    _RNG_TRACKER.reset()
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)
    else:
        torch.manual_seed(seed)
    _RNG_TRACKER.add(_MODEL_PARALLEL_RNG, tp_seed)


def split_tensor_into_1d_equal_chunks(tensor: torch.Tensor) -> torch.Tensor:
    """This rank's 1/tp slice of the flattened tensor (distributed activation checkpoints)."""
    data = tensor.reshape(-1)
    n = data.numel() // get_tensor_model_parallel_world_size()
    start = n * get_tensor_model_parallel_rank()
    return data[start:start + n]


def gather_split_1d_tensor(tensor: torch.Tensor) -> torch.Tensor:
    world = get_tensor_model_parallel_world_size()
    if world == 1:
        return tensor
    out = torch.empty(world * tensor.numel(), dtype=tensor.dtype, device=tensor.device)
    dist.all_gather_into_tensor(out, tensor.contiguous(), group=get_tensor_model_parallel_group())
    return out
