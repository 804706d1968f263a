"""Tensor-parallel building blocks: vocab-parallel embedding, column- and
row-parallel linear layers.

Weight layouts and semantics follow the reference
(metaseq/modules/megatron/mpu/layers.py: VocabParallelEmbedding :144-250,
ColumnParallelLinear :386-536, RowParallelLinear :539-676): column-parallel
weights are ``[out/p, in]``, row-parallel weights ``[out, in/p]``; with
``skip_bias_add`` the bias is returned instead of added so the caller can add it
after the tensor-parallel reduction; under sequence parallelism the
column-parallel input is all-gathered along the first dimension and the
row-parallel output reduce-scattered.

Initialisation: ``use_cpu_initialization`` builds the full master weight on
every rank and keeps this rank's slice (:61-101), otherwise the slice is drawn
directly inside the tensor-parallel RNG fork (:50-58).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from metaseq_b200.ops import autograd as ops_ag
from metaseq_b200.ops import functional as ops_f

from . import mappings, mpu


def _init_partition(weight: torch.Tensor, full_shape, partition_dim: int, init_method: Callable, cpu_init: bool,
                    stride: int = 1, dtype=None):
    """Fills ``weight`` (this rank's partition) from ``init_method``."""
    world = mpu.get_tensor_model_parallel_world_size()
    with torch.no_grad():
        if world == 1:
            if cpu_init and weight.device.type != "cpu":
                master = torch.empty(full_shape, dtype=torch.float32)
                init_method(master)
                weight.copy_(master)
            else:
                init_method(weight)
            return
        if cpu_init:
            master = torch.empty(full_shape, dtype=torch.float32)
            init_method(master)
            per = full_shape[partition_dim] // world
            per_stride = per // stride
            pieces = torch.split(master, per_stride, dim=partition_dim)
            rank = mpu.get_tensor_model_parallel_rank()
            mine = pieces[rank::world]
            weight.copy_(torch.cat(mine, dim=partition_dim))
        else:
            with mpu.get_cuda_rng_tracker().fork():
                init_method(weight)


class VocabParallelEmbedding(nn.Module):
    """Embedding whose rows (vocabulary) are split across tensor-parallel ranks; tokens
    outside this rank's range contribute zero and the partial results are all-reduced."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None,
                 init_method: Callable = nn.init.xavier_normal_, use_cpu_initialization: bool = True, dtype=None,
                 device=None):
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.padding_idx = padding_idx
        world = mpu.get_tensor_model_parallel_world_size()
        self.vocab_start_index, self.vocab_end_index = mpu.vocab_range(
            num_embeddings, mpu.get_tensor_model_parallel_rank(), world)
        self.num_embeddings_per_partition = self.vocab_end_index - self.vocab_start_index
        self.weight = nn.Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim, dtype=dtype,
                                               device=device))
        _init_partition(self.weight, (num_embeddings, embedding_dim), 0, init_method, use_cpu_initialization)
        if padding_idx is not None and self.vocab_start_index <= padding_idx < self.vocab_end_index:
            with torch.no_grad():
                self.weight[padding_idx - self.vocab_start_index].zero_()
        mpu.set_tensor_model_parallel_attributes(self.weight, world > 1, 0, 1)

    def forward(self, tokens):
        world = mpu.get_tensor_model_parallel_world_size()
        if world > 1:
            mask = (tokens < self.vocab_start_index) | (tokens >= self.vocab_end_index)
            local = (tokens - self.vocab_start_index).masked_fill(mask, 0)
        else:
            mask, local = None, tokens
        out = TF.embedding(local, self.weight, self.padding_idx if world == 1 else None)
        if mask is not None:
            out = out.masked_fill(mask.unsqueeze(-1), 0.0)
            out = mappings.reduce_from_tensor_model_parallel_region(out)
        return out


def _linear(x, weight, bias=None):
    if ops_f.use_kernels(x) and x.dtype == weight.dtype:
        return ops_ag.linear(x, weight, bias)
    return TF.linear(x, weight, bias)


def _mm(a, b, a_t=False, b_t=False):
    """``op(a) @ op(b)`` on 2-D operands: the tcgen05 GEMM on a GPU with 16-bit operands, ``torch.matmul`` elsewhere."""
    if ops_f.use_kernels(a) and a.dtype == b.dtype:
        # functional.gemm computes a @ b^T for row-major operands; the flags select the transposed reads
        return ops_f.gemm(a, b, a_mn=a_t, b_mn=not b_t)
    return (a.t() if a_t else a) @ (b.t() if b_t else b)


class LinearWithGradAccumulationAndAsyncCommunication(torch.autograd.Function):
    """Column-parallel product whose backward pass hides its collective behind the weight-gradient GEMM
    (reference: metaseq/modules/megatron/mpu/layers.py:253-383).

    Forward: under sequence parallelism the rows of ``x`` are gathered over the tensor-parallel group first;
    ``y = x W^T + b``.  Backward: the gathered input is rebuilt (asynchronously, behind the data-gradient product),
    then the data gradient's all-reduce (``async_grad_allreduce``) or reduce-scatter (sequence parallelism) is
    started, the weight gradient is computed while it runs, and the handle is waited on last.  With
    ``gradient_accumulation_fusion`` the weight gradient is added into ``weight.main_grad`` (fp32) and ``None`` is
    returned for it.  The fused decoder layer does the same overlap inside its GEMM kernels over peer memory; this
    function is the library-collective form for stand-alone column-parallel layers."""

    @staticmethod
    def forward(ctx, x, weight, bias, gradient_accumulation_fusion, async_grad_allreduce, sequence_parallel):
        assert not (async_grad_allreduce and sequence_parallel), "sequence parallelism reduce-scatters instead"
        ctx.save_for_backward(x, weight)
        ctx.use_bias = bias is not None
        ctx.flags = (bool(gradient_accumulation_fusion), bool(async_grad_allreduce), bool(sequence_parallel))
        total = mappings.gather_along_first_dim(x) if sequence_parallel else x
        y = _mm(total.reshape(-1, total.shape[-1]), weight, b_t=True).view(*total.shape[:-1], weight.shape[0])
        return y + bias if bias is not None else y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        fuse_accumulation, async_allreduce, sequence_parallel = ctx.flags
        world = mpu.get_tensor_model_parallel_world_size()
        group = mpu.get_tensor_model_parallel_group()
        dy = dy.contiguous()
        dy2 = dy.view(-1, dy.shape[-1])
        pending_gather = None
        if sequence_parallel and world > 1:
            total = torch.empty((x.shape[0] * world, *x.shape[1:]), dtype=x.dtype, device=x.device)
            pending_gather = torch.distributed.all_gather_into_tensor(total, x.contiguous(), group=group, async_op=True)
        else:
            total = x
        dx = _mm(dy2, weight).view(*dy.shape[:-1], weight.shape[1])
        pending, finish = None, None
        if world > 1 and async_allreduce:
            pending = torch.distributed.all_reduce(dx, group=group, async_op=True)
        elif world > 1 and sequence_parallel:
            pending, finish = mappings.start_reduce_scatter_along_first_dim(dx)
        if pending_gather is not None:
            pending_gather.wait()
        total2 = total.reshape(-1, total.shape[-1])
        if fuse_accumulation:
            weight.main_grad.addmm_(dy2.t().float(), total2.float())
            dw = None
        else:
            dw = _mm(dy2, total2, a_t=True)
        db = dy2.sum(dim=0) if ctx.use_bias else None
        if pending is not None:
            pending.wait()
        if finish is not None:
            dx = finish()
        return dx, dw, db, None, None, None


class ColumnParallelLinear(nn.Module):
    """``Y = X A^T + b`` with A split along its output dimension: ``A = [A_1; ...; A_p]``."""

    def __init__(self, input_size: int, output_size: int, bias: bool = True, gather_output: bool = True,
                 init_method: Callable = nn.init.xavier_normal_, stride: int = 1, skip_bias_add: bool = False,
                 use_cpu_initialization: bool = True, dtype=None, device=None, sequence_parallel: bool = False,
                 init_method_bias: Optional[Callable] = None, keep_master_weight_for_test: bool = False,
                 no_async_tensor_model_parallel_allreduce: bool = True, gradient_accumulation_fusion: bool = False):
        """The last four arguments are the reference's (metaseq/modules/megatron/mpu/layers.py:386-470):
        ``init_method_bias`` fills the bias (zeros without it); the others select library-collective variants
        there and are accepted here without effect (``LinearWithGradAccumulationAndAsyncCommunication`` is the
        stand-alone form of those variants)."""
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.gather_output = gather_output
        self.skip_bias_add = skip_bias_add
        self.sequence_parallel = sequence_parallel
        world = mpu.get_tensor_model_parallel_world_size()
        self.output_size_per_partition = mpu.divide(output_size, world)
        self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, input_size, dtype=dtype, device=device))
        _init_partition(self.weight, (output_size, input_size), 0, init_method, use_cpu_initialization, stride)
        mpu.set_tensor_model_parallel_attributes(self.weight, world > 1, 0, stride)
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, dtype=dtype, device=device))
            mpu.set_tensor_model_parallel_attributes(self.bias, world > 1, 0, stride)
            if init_method_bias is not None:
                with torch.no_grad():
                    init_method_bias(self.bias)
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        if self.sequence_parallel:
            xin = mappings.gather_from_sequence_parallel_region(x, True)
        else:
            xin = mappings.copy_to_tensor_model_parallel_region(x)
        bias = self.bias if not self.skip_bias_add else None
        out = _linear(xin, self.weight, bias)
        if self.gather_output:
            assert not self.sequence_parallel
            out = mappings.gather_from_tensor_model_parallel_region(out)
        return out, (self.bias if self.skip_bias_add else None)


class RowParallelLinear(nn.Module):
    """``Y = X A^T + b`` with A split along its input dimension and X split to match."""

    def __init__(self, input_size: int, output_size: int, bias: bool = True, input_is_parallel: bool = False,
                 init_method: Callable = nn.init.xavier_normal_, stride: int = 1, skip_bias_add: bool = False,
                 use_cpu_initialization: bool = True, dtype=None, device=None, sequence_parallel: bool = False,
                 keep_master_weight_for_test: bool = False, gradient_accumulation_fusion: bool = False):
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.input_is_parallel = input_is_parallel
        self.skip_bias_add = skip_bias_add
        self.sequence_parallel = sequence_parallel
        world = mpu.get_tensor_model_parallel_world_size()
        self.input_size_per_partition = mpu.divide(input_size, world)
        self.weight = nn.Parameter(torch.empty(output_size, self.input_size_per_partition, dtype=dtype, device=device))
        _init_partition(self.weight, (output_size, input_size), 1, init_method, use_cpu_initialization, stride)
        mpu.set_tensor_model_parallel_attributes(self.weight, world > 1, 1, stride)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, dtype=dtype, device=device))
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        xin = x if self.input_is_parallel else mappings.scatter_to_tensor_model_parallel_region(x)
        part = _linear(xin, self.weight, None)
        if self.sequence_parallel:
            out = mappings.reduce_scatter_to_sequence_parallel_region(part)
        else:
            out = mappings.reduce_from_tensor_model_parallel_region(part)
        if self.skip_bias_add:
            return out, self.bias
        if self.bias is not None:
            out = out + self.bias
        return out, None
