"""Tensor-parallel random state: the RNG tracker (default stream seeded with ``seed``, tensor-parallel stream
with ``seed + 2718 + tp_rank``) and the 1-D split / gather used by distributed activation checkpointing
(reference: metaseq/modules/megatron/mpu/random.py:60-220).  The implementations live in ``mpu``."""
from .mpu import (  # noqa: F401
    CudaRNGStatesTracker,
    RNGStatesTracker,
    gather_split_1d_tensor,
    get_cuda_rng_tracker,
    model_parallel_cuda_manual_seed,
    split_tensor_into_1d_equal_chunks,
)
