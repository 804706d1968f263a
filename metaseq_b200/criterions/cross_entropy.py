"""Token-level cross entropy, summed over the batch (reference:
metaseq/criterions/cross_entropy.py:40-136).  On a GPU with 16-bit logits the loss and its
gradient come from one fused kernel that overwrites the logits in place, so fp32
log-probabilities of shape ``[B*T, V]`` are never materialised."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as TF

from metaseq_b200.dataclass.configs import MetaseqDataclass
from metaseq_b200.logging import metrics
from metaseq_b200.ops import autograd as ops_ag
from metaseq_b200.ops import functional as ops_f

from . import register_criterion
from .base_criterion import BaseCriterion


@dataclass
class CrossEntropyCriterionConfig(MetaseqDataclass):
    pass


def nll_loss_sum(logits, target, ignore_index, row_stats=None):
    """Summed NLL of ``[N, V]`` logits.  ``row_stats``: the softmax pieces left by the logits product
    (``ops.autograd.linear(..., row_stats=True)``), which lift the kernel's limit on the vocabulary size."""
    if ops_f.use_kernels(logits) and logits.shape[-1] % 8 == 0 and \
            (row_stats is not None or logits.shape[-1] * 2 <= 200 * 1024):
        if row_stats is not None:
            logits._msq_row_stats = row_stats
        return ops_ag.cross_entropy_sum(logits, target, ignore_index)
    lprobs = TF.log_softmax(logits, dim=-1, dtype=torch.float32)
    return TF.nll_loss(lprobs, target, ignore_index=ignore_index, reduction="sum")


_GATHER_ABOVE = 2e9  # elements


def nll_loss(lprobs, target, ignore_index=None, reduction: str = "mean"):
    """NLL from log-probabilities.  ``torch.nn.functional.nll_loss`` below 2e9 elements; above that (where its
    index arithmetic overflows) a gather, with ignored targets contributing zero
    (metaseq/criterions/cross_entropy.py:15-37)."""
    if reduction not in ("mean", "sum", "none"):
        raise NotImplementedError(reduction)
    if lprobs.numel() < _GATHER_ABOVE:
        kw = {} if ignore_index is None else {"ignore_index": ignore_index}
        return TF.nll_loss(lprobs, target, reduction=reduction, **kw)
    index = target.unsqueeze(-1) if target.dim() == lprobs.dim() - 1 else target
    picked = -lprobs.gather(dim=-1, index=index).squeeze(-1)
    if ignore_index is not None:
        picked = picked.masked_fill(index.squeeze(-1).eq(ignore_index), 0.0)
    if reduction == "mean":
        return picked.mean()
    return picked.sum() if reduction == "sum" else picked


@register_criterion("cross_entropy", dataclass=CrossEntropyCriterionConfig)
class CrossEntropyCriterion(BaseCriterion):
    def __init__(self, task):
        super().__init__(task)

    def forward(self, model, sample, reduce=True):
        net_output = model(**sample["net_input"])
        loss, _ = self.compute_loss(model, net_output, sample, reduce=reduce)
        sample_size = sample["ntokens"]
        logging_output = {
            "loss": loss.data,
            "ntokens": sample["ntokens"],
            "nsentences": sample["target"].size(0),
            "sample_size": sample_size,
        }
        extra = net_output[1] if isinstance(net_output, (tuple, list)) and len(net_output) > 1 else {}
        if isinstance(extra, dict):
            if extra.get("tok_emb") is not None and not getattr(self, "_skip_norm_logging", False):
                with torch.no_grad():
                    emb = extra["tok_emb"]
                    logging_output["tok_norm"] = emb.detach().float().norm(dim=-1).mean().data
        return loss, sample_size, logging_output

    def compute_loss(self, model, net_output, sample, reduce=True):
        logits = net_output[0]
        target = model.get_targets(sample, net_output).reshape(-1)
        loss = nll_loss_sum(logits.reshape(-1, logits.size(-1)), target, self.padding_idx)
        return loss, loss

    @staticmethod
    def reduce_metrics(logging_outputs) -> None:
        loss_sum = sum(float(log.get("loss", 0)) for log in logging_outputs)
        ntokens = sum(float(log.get("ntokens", 0)) for log in logging_outputs)
        sample_size = sum(float(log.get("sample_size", 0)) for log in logging_outputs)
        for k in ("tok_norm", "pos_norm", "emb_norm", "actv_norm"):
            vals = [float(log[k]) for log in logging_outputs if k in log]
            if vals:
                metrics.log_scalar(k, sum(vals) / len(vals), round=3)
        metrics.log_scalar("loss", loss_sum / max(sample_size, 1) / math.log(2), sample_size, round=3)
        metrics.log_derived("ppl", lambda meters: _ppl(meters["loss"].avg))

    @staticmethod
    def logging_outputs_can_be_summed() -> bool:
        return True


def _ppl(loss, base=2):
    if loss is None:
        return 0.0
    try:
        return round(float(base ** loss), 2)
    except OverflowError:
        return float("inf")
