"""Cross entropy on vocabulary-sharded logits: the model keeps ``[B, T, V/p]`` on each
tensor-parallel rank and the loss is assembled with reductions over the group (reference:
metaseq/criterions/vocab_parallel_cross_entropy.py:15-110).  Sample size is the number of
non-pad target tokens."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from metaseq_b200.dataclass.configs import MetaseqDataclass
from metaseq_b200.logging import metrics
from metaseq_b200.parallel import mpu
from metaseq_b200.parallel.cross_entropy import vocab_parallel_cross_entropy

from . import register_criterion
from .base_criterion import BaseCriterion
from .cross_entropy import _ppl, nll_loss_sum


@dataclass
class VocabParallelCrossEntropyConfig(MetaseqDataclass):
    pass


@register_criterion("vocab_parallel_cross_entropy", dataclass=VocabParallelCrossEntropyConfig)
class VocabParallelCrossEntropyCriterion(BaseCriterion):
    def __init__(self, task):
        super().__init__(task)

    def forward(self, model, sample, reduce=True):
        target = sample["target"]
        # Non-pad target count comes from the collater (computed on the host before the batch is
        # copied to the device), so no device-to-host sync is needed here.
        has_pad = True
        net_output = model(**sample["net_input"])
        logits = net_output[0]
        row_stats = getattr(logits, "_msq_row_stats", None)  # left by the logits product's epilogue
        if mpu.get_tensor_model_parallel_world_size() == 1:
            loss = nll_loss_sum(logits.reshape(-1, logits.size(-1)), target.reshape(-1), self.padding_idx, row_stats)
        else:
            from metaseq_b200.parallel.cross_entropy import fused_vocab_parallel_cross_entropy_ok

            if fused_vocab_parallel_cross_entropy_ok(logits):
                per_tok = vocab_parallel_cross_entropy(logits, target, self.padding_idx, row_stats)  # in place
            else:
                per_tok = vocab_parallel_cross_entropy(logits.float(), target)
            if has_pad:
                per_tok = per_tok * (target != self.padding_idx)
            loss = per_tok.sum()
        ntok_target = sample.get("ntokens_target", sample["ntokens"])
        logging_output = {
            "loss": loss.data,
            "ntokens": sample["ntokens"],
            "nsentences": target.size(0),
            "sample_size": ntok_target,
        }
        if "src_tokens" in sample["net_input"] and hasattr(self.task, "eod"):
            logging_output["ndocseps"] = (target == self.task.eod).sum()
        extra = net_output[1] if len(net_output) > 1 and isinstance(net_output[1], dict) else {}
        for kind, total in (extra.get("norm_sums") or {}).items():
            logging_output[f"{kind}_norm"] = total  # sum over tokens of the L2 norm; averaged in reduce_metrics
        return loss, ntok_target, logging_output

    @staticmethod
    def reduce_metrics(logging_outputs) -> None:
        loss_sum = sum(float(log.get("loss", 0)) for log in logging_outputs)
        sample_size = sum(float(log.get("sample_size", 0)) for log in logging_outputs)
        ntokens = sum(float(log.get("ntokens", 0)) for log in logging_outputs)
        for kind in ("actv", "pos", "tok", "emb"):
            key = f"{kind}_norm"
            if any(key in log for log in logging_outputs):
                metrics.log_scalar(key, sum(log.get(key, 0) for log in logging_outputs) / max(ntokens, 1), round=3)
        if any("ndocseps" in log for log in logging_outputs):
            nsentences = sum(float(log.get("nsentences", 0)) for log in logging_outputs)
            ndocseps = sum(log.get("ndocseps", 0) for log in logging_outputs)
            metrics.log_scalar("docsperex", (ndocseps + nsentences) / max(nsentences, 1))
        metrics.log_scalar("loss", loss_sum / max(sample_size, 1) / math.log(2), sample_size, round=3)
        metrics.log_derived("ppl", lambda meters: _ppl(meters["loss"].avg))

    @staticmethod
    def logging_outputs_can_be_summed() -> bool:
        return True
