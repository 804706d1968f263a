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


def vocab_parallel_cross_entropy(vocab_parallel_logits, target):
    """Per-token NLL for ``[..., V/p]`` logits and global-vocabulary targets."""
    return _VocabParallelCrossEntropy.apply(vocab_parallel_logits, target)
