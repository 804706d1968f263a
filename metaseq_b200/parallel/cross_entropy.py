"""Cross entropy over vocabulary-parallel logits.

Each tensor-parallel rank holds ``[..., V/p]`` logits.  The loss needs three
cross-rank reductions per token: the max logit, the target logit (owned by one
rank) and the sum of exponentials (reference:
metaseq/modules/megatron/mpu/cross_entropy.py:19-109, three separate
all-reduces).  Here the max is one MAX all-reduce and the other two travel
together in a single SUM all-reduce of a ``[rows, 2]`` buffer.  As in the
reference the local logits buffer is overwritten with the softmax so the
backward needs no second pass over the vocabulary.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import mpu


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, vocab_parallel_logits, target):
        group = mpu.get_tensor_model_parallel_group()
        world = mpu.get_tensor_model_parallel_world_size()
        rank = mpu.get_tensor_model_parallel_rank()
        # The buffer is overwritten in place (it becomes the softmax).  Working on the ``.data`` alias keeps
        # autograd's version counter of the incoming tensor untouched, which matters when that tensor is
        # itself the (view) output of another custom function.
        logits = vocab_parallel_logits.data
        part = logits.shape[-1]
        start, end = rank * part, (rank + 1) * part

        logits_max = logits.max(dim=-1)[0]
        if world > 1:
            dist.all_reduce(logits_max, op=dist.ReduceOp.MAX, group=group)
        logits.sub_(logits_max.unsqueeze(-1))

        mask = (target < start) | (target >= end)
        local_t = (target - start).masked_fill(mask, 0)
        l2 = logits.view(-1, part)
        rows = torch.arange(l2.shape[0], device=l2.device)
        picked = l2[rows, local_t.view(-1)].clone().view_as(target)
        picked.masked_fill_(mask, 0.0)

        torch.exp(logits, out=logits)
        pair = torch.stack([picked, logits.sum(dim=-1)], dim=-1).contiguous()
        if world > 1:
            dist.all_reduce(pair, group=group)
        picked, sum_exp = pair[..., 0], pair[..., 1]
        loss = torch.log(sum_exp) - picked
        logits.div_(sum_exp.unsqueeze(-1))
        ctx.save_for_backward(logits, mask, local_t)
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        softmax, mask, local_t = ctx.saved_tensors
        part = softmax.shape[-1]
        grad = softmax
        g2 = grad.view(-1, part)
        rows = torch.arange(g2.shape[0], device=g2.device)
        g2[rows, local_t.view(-1)] -= 1.0 - mask.view(-1).to(g2.dtype)
        grad.mul_(grad_output.unsqueeze(-1))
        return grad, None


class _FusedVocabParallelCrossEntropy(torch.autograd.Function):
    """Kernel path for 16-bit logits on a GPU.  Every rank needs, per row, the (max, sum-exp, target logit) of each
    rank's vocabulary slice.  Where the logits product left its row statistics (``row_stats``) one small kernel folds
    them and, with the fused communication backend, stores the triple straight into every peer's exchange table over
    NVLink; the kernel that writes the loss and overwrites the logits with the gradient polls its own table.  Without
    row statistics one kernel reads the logits for the triples, and without the fused backend they travel in one
    small NCCL all-reduce.  fp32 logits are never materialised."""

    @staticmethod
    def forward(ctx, logits, target, ignore_index, row_stats=None):
        from metaseq_b200.ops import _lib
        from metaseq_b200.ops import autograd as ops_ag
        from metaseq_b200.parallel import symm

        group = mpu.get_tensor_model_parallel_group()
        world = mpu.get_tensor_model_parallel_world_size()
        rank = mpu.get_tensor_model_parallel_rank()
        V = logits.shape[-1]
        l2 = logits.data.reshape(-1, V)
        rows = l2.shape[0]
        tgt = target.reshape(-1).contiguous()
        lib = _lib.kernels()
        bf = int(logits.dtype == torch.bfloat16)
        ctx.pre_scaled = ops_ag.upstream_grad_hint()
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        exchange = symm.get_ce_exchange(group, logits.device, rows) if row_stats is not None else None
        if exchange is not None:
            tables, mine, epoch = exchange.next()
            rc = lib.msq_ce_merge_rowstats(_lib.ptr(row_stats[0]), _lib.ptr(row_stats[1]), row_stats[0].shape[0], rows,
                                           _lib.ptr(l2), l2.stride(0), _lib.ptr(tgt), V, rank * V, None, tables, world,
                                           rank, exchange.rows_cap, epoch, bf, _lib.stream_ptr())
            _lib.check_rc(rc, "msq_ce_merge_rowstats")
            import ctypes

            rc = lib.msq_vp_ce_finish_exchanged(_lib.ptr(l2), l2.stride(0), _lib.ptr(tgt), ctypes.c_void_p(mine), world,
                                                exchange.rows_cap, epoch, _lib.ptr(loss), rows, V, rank * V,
                                                int(ignore_index), ctx.pre_scaled, bf,
                                                _lib.ptr(_lib.status_word(logits.device)), _lib.stream_ptr())
            _lib.check_rc(rc, "msq_vp_ce_finish_exchanged")
            _note_exchange_once(world, rows)
        else:
            stats = torch.zeros((world, rows, 3), dtype=torch.float32, device=logits.device)
            if row_stats is not None:
                rc = lib.msq_ce_merge_rowstats(_lib.ptr(row_stats[0]), _lib.ptr(row_stats[1]), row_stats[0].shape[0],
                                               rows, _lib.ptr(l2), l2.stride(0), _lib.ptr(tgt), V, rank * V,
                                               _lib.ptr(stats[rank]), None, 1, 0, rows, 0, bf, _lib.stream_ptr())
                _lib.check_rc(rc, "msq_ce_merge_rowstats")
            else:
                rc = lib.msq_vp_ce_partial(_lib.ptr(l2), l2.stride(0), _lib.ptr(tgt), _lib.ptr(stats[rank]), rows, V,
                                           rank * V, bf, _lib.stream_ptr())
                _lib.check_rc(rc, "msq_vp_ce_partial")
            if world > 1:
                tp = symm.get_tp_comm(group, logits.device, 1, 8, logits.dtype) if symm.comm_backend() == "fused" else None
                if tp is not None:
                    tp.comm.all_reduce(stats.view(-1))
                else:
                    dist.all_reduce(stats, group=group)
            rc = lib.msq_vp_ce_finish(_lib.ptr(l2), l2.stride(0), _lib.ptr(tgt), _lib.ptr(stats), world, _lib.ptr(loss),
                                      rows, V, rank * V, int(ignore_index), ctx.pre_scaled, bf, _lib.stream_ptr())
            _lib.check_rc(rc, "msq_vp_ce_finish")
        ctx.save_for_backward(l2)
        ctx.shape = logits.shape
        return loss.view(target.shape)

    @staticmethod
    def backward(ctx, grad_output):
        (grad,) = ctx.saved_tensors  # (softmax - onehot) * pre_scaled, zero rows where the target is ignored
        from metaseq_b200.ops import functional as ops_f

        # in place: the saved tensor is the logits buffer, which nothing else reads after the loss.  Rows whose
        # incoming factor equals the one already applied are left alone.
        ops_f.scale_rows_(grad, grad_output, ref=ctx.pre_scaled)
        return grad.view(ctx.shape), None, None, None


_EXCHANGE_NOTED = [False]


def _note_exchange_once(world, rows):
    if not _EXCHANGE_NOTED[0]:
        _EXCHANGE_NOTED[0] = True
        import logging

        logging.getLogger(__name__).info(
            "vocab-parallel cross entropy: row statistics from the logits GEMM epilogue, exchanged over peer memory "
            "(%d ranks, %d rows)", world, rows)


def fused_vocab_parallel_cross_entropy_ok(logits) -> bool:
    from metaseq_b200.ops import functional as F

    return (logits.is_cuda and logits.dtype in (torch.float16, torch.bfloat16) and F.use_kernels(logits)
            and logits.shape[-1] % 8 == 0 and logits.is_contiguous())


def vocab_parallel_cross_entropy(vocab_parallel_logits, target, ignore_index: int = -100, row_stats=None):
    """Per-token NLL for ``[..., V/p]`` logits and global-vocabulary targets.  16-bit logits on a GPU take the
    kernel path (rows whose target equals ``ignore_index`` get zero loss and gradient there); otherwise the
    PyTorch implementation, which needs fp32 logits and leaves the masking of ignored targets to the caller.
    ``row_stats`` (default: the ``_msq_row_stats`` attribute of the logits): the softmax pieces that the logits
    product computed in its epilogue."""
    if fused_vocab_parallel_cross_entropy_ok(vocab_parallel_logits):
        if row_stats is None:
            row_stats = getattr(vocab_parallel_logits, "_msq_row_stats", None)
        return _FusedVocabParallelCrossEntropy.apply(vocab_parallel_logits, target, ignore_index, row_stats)
    return _VocabParallelCrossEntropy.apply(vocab_parallel_logits, target)
