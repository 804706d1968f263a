"""Config dataclasses: the single source of truth for every command-line flag.

Flag names, groups and defaults follow the reference
(metaseq/dataclass/configs.py:82-801) so that command lines written for
``metaseq-train`` keep working.  The machinery is different: the reference
composes these through hydra/omegaconf; here they are plain dataclasses with an
``opt()`` field helper, converted to argparse flags and to a nested
attribute-dict config by ``metaseq_b200.dataclass.utils``.

A field declared with ``link="group.name"`` mirrors another field (the
reference's ``II("group.name")`` interpolation) and gets no flag of its own.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass, field, fields
from typing import Any, List, Optional

from .constants import (
    CLIP_GRAD_NORM_TYPE_CHOICES,
    DATASET_IMPL_CHOICES,
    DDP_BACKEND_CHOICES,
    LOG_FORMAT_CHOICES,
    TASK_DDP_BACKEND_CHOICES,
)


def opt(default=None, help: str = "", *, choices=None, alias=None, link=None, const=None, factory=None):
    """Declare one config field / command-line flag."""
    meta = {"help": help}
    if choices is not None:
        meta["choices"] = tuple(choices)
    if alias is not None:
        meta["argparse_alias"] = alias
    if link is not None:
        meta["link"] = link
    if const is not None:
        meta["argparse_const"] = const
    if factory is not None:
        return field(default_factory=factory, metadata=meta)
    return field(default=default, metadata=meta)


@dataclass
class MetaseqDataclass:
    """Base for all config groups."""

    _name: Optional[str] = None

    @staticmethod
    def name():
        return None

    def positional_args(self):
        """Flags that the command line takes by position rather than by ``--name``."""
        return ["data"]

    def field_names(self):
        return [f.name for f in fields(self) if not f.name.startswith("_")]

    def meta(self, attr: str, key: str, default=None):
        return self.__dataclass_fields__[attr].metadata.get(key, default)

    def to_dict(self) -> dict:
        return {k: getattr(self, k) for k in self.field_names()}


def _device_count() -> int:
    try:
        import torch

        return max(1, torch.cuda.device_count())
    except Exception:
        return 1


@dataclass
class CommonConfig(MetaseqDataclass):
    log_interval: int = opt(100, "number of batches between two progress lines")
    log_format: Optional[str] = opt(None, "how progress is printed", choices=LOG_FORMAT_CHOICES)
    log_file: Optional[str] = opt(None, "metrics are also appended to this file")
    tensorboard_logdir: Optional[str] = opt(None, "directory for tensorboard event files")
    aim_repo: Optional[str] = opt(None, "location of the Aim repository to log to")
    aim_run_hash: Optional[str] = opt(None, "hash of an existing Aim run to continue")
    wandb_project: Optional[str] = opt(None, "project name on Weights and Biases")
    azureml_logging: Optional[bool] = opt(False, "send scalars to the AzureML run context")
    seed: int = opt(1, "seed of every random number generator")
    seed_per_rank: bool = opt(False, "offset the seed by the rank")
    cpu: bool = opt(False, "run on the host even when a GPU is present")
    fp16: bool = opt(False, "half-precision weights and activations with fp32 master weights")
    memory_efficient_fp16: bool = opt(False, "half precision without an fp32 master copy (the optimizer "
                                             "computes in fp32 internally); turns --fp16 on")
    bf16: bool = opt(False, "bfloat16 weights and activations")
    fp16_no_flatten_grads: bool = opt(False, "keep half-precision gradients as separate tensors")
    fp16_init_scale: int = opt(4, "loss scale at the start")
    fp16_scale_window: Optional[int] = opt(256, "overflow-free updates after which the loss scale doubles")
    fp16_scale_tolerance: float = opt(0.0, "share of updates that may overflow before the loss scale is halved")
    min_loss_scale: float = opt(2 ** -5, "training stops when the loss scale falls below this")
    threshold_loss_scale: Optional[float] = opt(None, "the loss scale is never lowered below this")
    user_dir: Optional[str] = opt(None, "python module with user-defined tasks, models or criterions to import")
    empty_cache_freq: int = opt(0, "release the CUDA caching allocator's blocks every N updates (0 = never)")
    all_gather_list_size: int = opt(16384, "byte size of the buffer for gathering python objects over ranks")
    model_parallel_size: int = opt(1, "tensor-parallel width (GPUs that share one model replica)")
    profile: bool = opt(False, "trace a few updates of rank 0 with the torch profiler")
    watchdog_timeout: float = opt(0.0, "seconds without a finished training step (or with a kernel reporting a "
                                       "timed-out wait) after which the host watchdog dumps all thread stacks and "
                                       "interrupts the run; 0 disables it")
    use_plasma_view: bool = opt(False, "keep dataset index and size arrays in shared memory")
    plasma_path: Optional[str] = opt("/tmp/plasma", "socket path of the shared-memory store")
    log_nvidia_smi: bool = opt(False, "add nvidia-smi memory readings to the training log")
    quiet_logs: Optional[bool] = opt(False, "leave per-parameter gradient / weight norms out of the log")
    log_param_stats: bool = opt(False, "log norm / max / zero share of every flat parameter and its gradient each "
                                       "update (a few hundred small reductions per update; off by default)")
    # additions of this framework
    kernel_backend: str = opt("auto", "operator backend: sm_100a kernels when possible (auto) or PyTorch/cuBLAS "
                              "ops everywhere (torch), which is the unfused baseline", choices=("auto", "torch"))
    strict_kernels: bool = opt(False, "raise when an operator on CUDA 16-bit tensors would leave the sm_100a "
                                      "kernels for PyTorch ops (unsupported head size, stride or alignment) "
                                      "instead of logging the fallback once")
    comm_backend: str = opt("fused", "collective path for FSDP / tensor parallel hot ops: in-kernel NVLink peer "
                            "access (fused) or NCCL calls (nccl)", choices=("fused", "nccl"))


@dataclass
class DistributedTrainingConfig(MetaseqDataclass):
    distributed_world_size: int = opt(factory=_device_count, help="number of ranks (one per GPU) over all nodes")
    distributed_rank: Optional[int] = opt(0, "this process's rank")
    distributed_backend: str = opt("nccl", "torch.distributed backend")
    distributed_init_method: Optional[str] = opt(None, "rendezvous URL, e.g. tcp://host:port")
    distributed_port: int = opt(-1, "rendezvous port when no URL is given")
    device_id: int = opt(0, "local GPU index (normally set by the launcher)", alias="--local_rank")
    distributed_no_spawn: bool = opt(False, "stay in one process although several GPUs are visible")
    ddp_backend: str = opt("pytorch_ddp", "data-parallel engine", choices=DDP_BACKEND_CHOICES)
    task_ddp_backend: str = opt("none", "data-parallel engine chosen by the task, if any",
                                choices=TASK_DDP_BACKEND_CHOICES)
    bucket_cap_mb: int = opt(25, "gradient bucket size in MB")
    fix_batches_to_gpus: bool = opt(False, "every rank keeps the same batches in every epoch")
    find_unused_parameters: bool = opt(False, "let DDP search for parameters without gradient")
    fast_stat_sync: bool = opt(False, "no effect (kept for old command lines)")
    broadcast_buffers: bool = opt(False, "synchronise module buffers over ranks every step")
    fp16: bool = opt(False, link="common.fp16")
    memory_efficient_fp16: bool = opt(False, link="common.memory_efficient_fp16")
    bf16: bool = opt(False, link="common.bf16")
    no_reshard_after_forward: bool = opt(False, "keep gathered parameters until backward (ZeRO-2 style)")
    fp32_reduce_scatter: bool = opt(False, "sum gradient shards in fp32")
    cpu_offload: bool = opt(False, "keep fp32 shards and optimizer state in host memory")
    use_sharded_state: Optional[bool] = opt(False, "checkpoints hold each rank's shard, not the full model")
    gradient_predivide_factor: Optional[float] = opt(None, "divide gradients by this before the reduce-scatter "
                                                           "and by world / this after")


@dataclass
class DatasetConfig(MetaseqDataclass):
    num_workers: int = opt(1, "data loader worker processes")
    num_workers_valid: int = opt(0, "data loader worker processes for validation")
    skip_invalid_size_inputs_valid_test: bool = opt(False, "drop evaluation samples outside the model's length "
                                                           "limits instead of failing")
    max_tokens: Optional[int] = opt(None, "token budget of one batch")
    batch_size: Optional[int] = opt(None, "samples per batch", alias="--max-sentences")
    required_batch_size_multiple: int = opt(8, "batch sizes are cut to a multiple of this")
    dataset_impl: Optional[str] = opt(None, "on-disk format of indexed datasets", choices=DATASET_IMPL_CHOICES)
    data_buffer_size: int = opt(10, "batches prefetched ahead of the training loop")
    skip_batches: str = opt("", "update ranges whose batches are read but not trained on, e.g. "
                                "'100-200,150-250'")
    train_subset: str = opt("train", "split to train on")
    valid_subset: str = opt("valid", "splits to validate on, comma separated")
    combine_valid_subsets: Optional[bool] = opt(None, "validate on the union of all valid* splits as one set",
                                                alias="--combine-val")
    ignore_unused_valid_subsets: Optional[bool] = opt(False, "valid* directories that are not listed are fine")
    validate_interval_updates: int = opt(0, "validate every N updates (0 = only at epoch ends)")
    validate_after_updates: int = opt(0, "no validation before update N")
    fixed_validation_seed: Optional[int] = opt(None, "reseed before every validation pass")
    disable_validation: bool = opt(False, "never validate")
    max_tokens_valid: Optional[int] = opt(None, "token budget of a validation batch",
                                          link="dataset.max_tokens")
    batch_size_valid: Optional[int] = opt(None, "samples per validation batch", link="dataset.batch_size",
                                          alias="--max-sentences-valid")
    max_valid_steps: Optional[int] = opt(None, "stop a validation pass after N batches", alias="--nval")
    gen_subset: str = opt("test", "split used for generation")
    num_shards: int = opt(1, "number of parts the generation set is cut into")
    shard_id: int = opt(0, "which of those parts this process takes")


@dataclass
class OptimizationConfig(MetaseqDataclass):
    max_epoch: int = opt(0, "last epoch (0 = no limit)")
    max_update: int = opt(0, "last update (0 = no limit)")
    clip_norm: float = opt(0.0, "gradient norm above which gradients are scaled down (0 = off)")
    clip_norm_type: Optional[str] = opt("l2", "norm used for clipping: l2, or inf for the largest absolute "
                                              "value",
                                        choices=CLIP_GRAD_NORM_TYPE_CHOICES)
    skip_gradient_update_on_clip_norm: bool = opt(False, "reject the batch when its gradient norm exceeds "
                                                         "--clip-norm")
    ewm_ratio_to_skip_batch: float = opt(-1, "skip a batch whose loss / ewm(loss) exceeds this ratio (-1 disables)")
    update_freq: List[int] = opt(factory=lambda: [1], help="micro-batches accumulated per update, one entry "
                                                           "per epoch")
    lr: List[float] = opt(factory=lambda: [0.25], help="peak learning rate, one entry per epoch (the last one "
                                                       "repeats)")


@dataclass
class CheckpointConfig(MetaseqDataclass):
    save_dir: str = opt("checkpoints", "directory for checkpoints")
    restore_file: str = opt("checkpoint_last.pt", "checkpoint to resume from (a name inside --save-dir or a "
                                                  "path)")
    finetune_from_model: Optional[str] = opt(None, "start from these weights with fresh optimizer, schedule, "
                                                   "meters and data position")
    reset_dataloader: bool = opt(False, "start the data from the beginning although the checkpoint has a "
                                        "position")
    reset_lr_scheduler: bool = opt(False, "ignore the schedule state of the checkpoint")
    reset_meters: bool = opt(False, "ignore the meters of the checkpoint")
    reset_optimizer: bool = opt(False, "ignore the optimizer state of the checkpoint")
    optimizer_overrides: str = opt("{}", "python dict of optimizer settings that replace the checkpoint's")
    save_interval_epochs: int = opt(1, "epochs between checkpoints")
    save_interval_updates: int = opt(0, "updates between checkpoints (each is followed by a validation pass)")
    local_save_interval_updates: int = opt(0, "updates between checkpoints that stay on local disk")
    save_last_checkpoint: bool = opt(True, "write checkpoint_last when training ends")
    keep_last_epochs: int = opt(-1, "older epoch checkpoints are deleted beyond this many (-1 = keep all)")
    keep_last_updates: int = opt(-1, "older update checkpoints are deleted beyond this many (-1 = keep all)")
    checkpoint_suffix: str = opt("", "inserted before .pt in checkpoint names")
    checkpoint_shard_count: int = opt(1, "files one checkpoint is split over")
    write_checkpoints_asynchronously: bool = opt(True, "serialise and write on a background thread",
                                                 alias="--save-async")
    cloud_upload_path: Optional[str] = opt(None, "blob-storage URL or nfs:<dir> that finished checkpoints are "
                                                 "moved to")
    nfs_eval_script_path: Optional[str] = opt(None, "script started on each checkpoint that has arrived on the "
                                                    "shared directory")
    nfs_eval_num_attempts: int = opt(10, "times to look for all parts of a checkpoint before giving up on its "
                                         "evaluation")
    nfs_eval_attempt_wait_minutes: int = opt(5, "minutes between those looks")
    nfs_eval_frequency: int = opt(5000, "only checkpoints whose update is a multiple of this are evaluated")
    cluster_env: str = opt("fair", "where the job runs: azure, aws, fair or rsc")
    model_parallel_size: int = opt(1, link="common.model_parallel_size")
    sequence_parallel: bool = opt(False, "shard LayerNorm / residual regions along the sequence across the "
                                  "tensor-parallel group (needs --model-parallel-size > 1)")


@dataclass
class GenerationConfig(MetaseqDataclass):
    beam: int = opt(5, "hypotheses kept per prompt")
    max_len_a: float = opt(0, "a in the length limit a * prompt length + b")
    max_len_b: int = opt(200, "b in the length limit a * prompt length + b")
    min_len: int = opt(1, "fewest tokens to generate")
    sampling: bool = opt(False, "draw tokens at random instead of taking the best")
    sampling_topp: float = opt(-1.0, "nucleus sampling: restrict to the most probable tokens whose mass "
                                     "reaches p")
    temperature: float = opt(1.0, "logits are divided by this before sampling")
    no_seed_provided: bool = opt(False, "set by the parser when --seed was not given")
    buffer_size: int = opt(0, "input lines read ahead in interactive mode")
    input: str = opt("-", "input file (- = standard input)")


@dataclass
class CommonEvalConfig(MetaseqDataclass):
    path: Optional[str] = opt(None, "checkpoint file(s), separated by colons")
    quiet: bool = opt(False, "print the final numbers only")
    model_overrides: str = opt("{}", "python dict of model settings that replace the checkpoint's")
    results_path: Optional[str] = opt(None, "where evaluation output is written, if anywhere")


@dataclass
class ReshardConfig(MetaseqDataclass):
    save_dir: Optional[str] = opt(None, "output directory")
    save_prefix: Optional[str] = opt("reshard", "outputs are named <save-dir>/<save-prefix>-shard<i>.pt")
    target_world_size: Optional[int] = opt(128, "largest number of GPUs the result must load on")
    do_pad: Optional[bool] = opt(False, "pad flat parameters so that the target world size divides them")


@dataclass
class EvalLMConfig(MetaseqDataclass):
    score_sequences: bool = opt(False, "score given sequences instead of a corpus")
    output_word_probs: bool = opt(False, "print every word with its log probability")
    output_word_stats: bool = opt(False, "print per-word counts and mean probabilities")
    context_window: int = opt(0, "tokens of preceding text that every scored token can see at least")
    softmax_batch: int = opt(sys.maxsize, "compute the softmax in pieces of this many positions")
    max_valid_steps: Optional[int] = opt(None, "stop after N batches", alias="--nval")


@dataclass
class EMAConfig(MetaseqDataclass):
    store_ema: bool = opt(False, "keep an exponential moving average of the weights")
    ema_decay: float = opt(0.9999, "weight of the old average in each update of it")
    ema_start_update: int = opt(0, "averaging begins after this many updates")
    ema_seed_model: Optional[str] = opt(None, "checkpoint that initialises the average")
    ema_update_freq: int = opt(1, "updates between two updates of the average")
    ema_fp32: bool = opt(False, "hold the average in fp32 whatever the model's type")


GROUPS = {
    "common": CommonConfig,
    "common_eval": CommonEvalConfig,
    "distributed_training": DistributedTrainingConfig,
    "dataset": DatasetConfig,
    "optimization": OptimizationConfig,
    "checkpoint": CheckpointConfig,
    "generation": GenerationConfig,
    "eval_lm": EvalLMConfig,
    "reshard": ReshardConfig,
    "ema": EMAConfig,
}
# groups filled from the component registries (a dataclass instance or a plain namespace)
COMPONENT_GROUPS = ("model", "task", "criterion", "optimizer", "lr_scheduler", "bpe", "tokenizer")


@dataclass
class MetaseqConfig(MetaseqDataclass):
    common: CommonConfig = field(default_factory=CommonConfig)
    common_eval: CommonEvalConfig = field(default_factory=CommonEvalConfig)
    distributed_training: DistributedTrainingConfig = field(default_factory=DistributedTrainingConfig)
    dataset: DatasetConfig = field(default_factory=DatasetConfig)
    optimization: OptimizationConfig = field(default_factory=OptimizationConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    generation: GenerationConfig = field(default_factory=GenerationConfig)
    eval_lm: EvalLMConfig = field(default_factory=EvalLMConfig)
    reshard: ReshardConfig = field(default_factory=ReshardConfig)
    ema: EMAConfig = field(default_factory=EMAConfig)
    model: Any = None
    task: Any = None
    criterion: Any = None
    optimizer: Any = None
    lr_scheduler: Any = None
    bpe: Any = None
    tokenizer: Any = None
