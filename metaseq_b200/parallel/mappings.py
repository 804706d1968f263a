"""Autograd-aware collectives over the tensor-parallel group.

Same set as the reference (metaseq/modules/megatron/mpu/mappings.py:179-332):
copy / reduce / scatter / gather along the last dimension for plain tensor
parallelism, and scatter / gather / reduce-scatter along the first (sequence)
dimension for sequence parallelism.  These are the NCCL (or gloo) forms used by
the modular path and as the baseline; the fused decoder layer replaces the hot
ones with in-kernel peer access.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import mpu


def _world():
    return mpu.get_tensor_model_parallel_world_size()


def _group():
    return mpu.get_tensor_model_parallel_group()


def _reduce(x):
    if _world() == 1:
        return x
    dist.all_reduce(x, group=_group())
    return x


def _split_last(x):
    w = _world()
    if w == 1:
        return x
    return x.chunk(w, dim=-1)[mpu.get_tensor_model_parallel_rank()].contiguous()


def _gather_last(x):
    w = _world()
    if w == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(w)]
    dist.all_gather(parts, x.contiguous(), group=_group())
    return torch.cat(parts, dim=-1).contiguous()


def _split_first(x):
    w = _world()
    if w == 1:
        return x
    assert x.shape[0] % w == 0, "first dimension must be divisible by the tensor-parallel size"
    n = x.shape[0] // w
    r = mpu.get_tensor_model_parallel_rank()
    return x[r * n:(r + 1) * n].contiguous()


def gather_along_first_dim(x):
    w = _world()
    if w == 1:
        return x
    out = torch.empty((x.shape[0] * w, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=_group())
    return out


def reduce_scatter_along_first_dim(x):
    w = _world()
    if w == 1:
        return x
    assert x.shape[0] % w == 0
    out = torch.empty((x.shape[0] // w, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=_group())
    return out


def start_reduce_scatter_along_first_dim(x):
    """Starts the reduce-scatter of ``x`` over the tensor-parallel group and returns ``(handle, finish)``:
    ``finish()`` gives this rank's rows once ``handle.wait()`` has returned.  Backends without a reduce-scatter
    (gloo) all-reduce in place and ``finish`` slices."""
    w = _world()
    assert w > 1 and x.shape[0] % w == 0
    x = x.contiguous()
    if dist.get_backend(_group()) == "gloo":
        handle = dist.all_reduce(x, group=_group(), async_op=True)
        return handle, lambda: _split_first(x)
    out = torch.empty((x.shape[0] // w, *x.shape[1:]), dtype=x.dtype, device=x.device)
    handle = dist.reduce_scatter_tensor(out, x, group=_group(), async_op=True)
    return handle, lambda: out


class _CopyToModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return _reduce(g.contiguous().clone() if _world() > 1 else g)


class _ReduceFromModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _reduce(x.contiguous().clone() if _world() > 1 else x)

    @staticmethod
    def backward(ctx, g):
        return g


class _ScatterToModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _split_last(x)

    @staticmethod
    def backward(ctx, g):
        return _gather_last(g)


class _GatherFromModelParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _gather_last(x)

    @staticmethod
    def backward(ctx, g):
        return _split_last(g)


class _ScatterToSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _split_first(x)

    @staticmethod
    def backward(ctx, g):
        return gather_along_first_dim(g)


class _GatherFromSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, to_model_parallel=True):
        ctx.to_model_parallel = to_model_parallel
        return gather_along_first_dim(x)

    @staticmethod
    def backward(ctx, g):
        if ctx.to_model_parallel:
            return reduce_scatter_along_first_dim(g), None
        return _split_first(g), None


class _ReduceScatterToSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return reduce_scatter_along_first_dim(x)

    @staticmethod
    def backward(ctx, g):
        return gather_along_first_dim(g)


def copy_to_tensor_model_parallel_region(x):
    return _CopyToModelParallelRegion.apply(x)


def reduce_from_tensor_model_parallel_region(x):
    return _ReduceFromModelParallelRegion.apply(x)


def scatter_to_tensor_model_parallel_region(x):
    return _ScatterToModelParallelRegion.apply(x)


def gather_from_tensor_model_parallel_region(x):
    return _GatherFromModelParallelRegion.apply(x)


def scatter_to_sequence_parallel_region(x):
    return _ScatterToSequenceParallelRegion.apply(x)


def gather_from_sequence_parallel_region(x, to_model_parallel=True):
    return _GatherFromSequenceParallelRegion.apply(x, to_model_parallel)


def reduce_scatter_to_sequence_parallel_region(x):
    return _ReduceScatterToSequenceParallelRegion.apply(x)
