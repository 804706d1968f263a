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
    log_interval: int = opt(100, "log progress every N batches")
    log_format: Optional[str] = opt(None, "log format to use", choices=LOG_FORMAT_CHOICES)
    log_file: Optional[str] = opt(None, "log file to copy metrics to")
    tensorboard_logdir: Optional[str] = opt(None, "path to save logs for tensorboard")
    aim_repo: Optional[str] = opt(None, "path to Aim repository")
    aim_run_hash: Optional[str] = opt(None, "Aim run hash")
    wandb_project: Optional[str] = opt(None, "Weights and Biases project name")
    azureml_logging: Optional[bool] = opt(False, "log scalars to AzureML context")
    seed: int = opt(1, "pseudo random number generator seed")
    seed_per_rank: bool = opt(False, "use different seed per rank")
    cpu: bool = opt(False, "use CPU instead of CUDA")
    fp16: bool = opt(False, "use FP16")
    memory_efficient_fp16: bool = opt(False, "use a memory-efficient version of FP16 training; implies --fp16")
    bf16: bool = opt(False, "use BF16 format")
    fp16_no_flatten_grads: bool = opt(False, "don't flatten FP16 grads tensor")
    fp16_init_scale: int = opt(4, "default FP16 loss scale")
    fp16_scale_window: Optional[int] = opt(256, "number of updates before increasing loss scale")
    fp16_scale_tolerance: float = opt(0.0, "pct of updates that can overflow before decreasing the loss scale")
    min_loss_scale: float = opt(2 ** -5, "minimum FP16 loss scale, after which training is stopped")
    threshold_loss_scale: Optional[float] = opt(None, "threshold FP16 loss scale from below")
    user_dir: Optional[str] = opt(None, "path to a python module containing custom extensions")
    empty_cache_freq: int = opt(0, "how often to clear the PyTorch CUDA cache (0 to disable)")
    all_gather_list_size: int = opt(16384, "number of bytes reserved for gathering stats from workers")
    model_parallel_size: int = opt(1, "total number of GPUs to parallelize model over")
    profile: bool = opt(False, "use pytorch profiler on the 6th step of rank 0")
    watchdog_timeout: float = opt(0.0, "seconds without a finished training step (or with a kernel reporting a "
                                       "timed-out wait) after which the host watchdog dumps all thread stacks and "
                                       "interrupts the run; 0 disables it")
    use_plasma_view: bool = opt(False, "store indices and sizes in shared memory")
    plasma_path: Optional[str] = opt("/tmp/plasma", "path to run plasma_store")
    log_nvidia_smi: bool = opt(False, "log output from nvidia-smi during training")
    quiet_logs: Optional[bool] = opt(False, "don't log per-parameter gnorm/pnorm stats")
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
    distributed_world_size: int = opt(factory=_device_count, help="total number of GPUs across all nodes")
    distributed_rank: Optional[int] = opt(0, "rank of the current worker")
    distributed_backend: str = opt("nccl", "distributed backend")
    distributed_init_method: Optional[str] = opt(None, "typically tcp://hostname:port used to establish the "
                                                 "initial connection")
    distributed_port: int = opt(-1, "port number (not required if using --distributed-init-method)")
    device_id: int = opt(0, "which GPU to use (usually configured automatically)", alias="--local_rank")
    distributed_no_spawn: bool = opt(False, "do not spawn multiple processes even if multiple GPUs are visible")
    ddp_backend: str = opt("pytorch_ddp", "DistributedDataParallel backend", choices=DDP_BACKEND_CHOICES)
    task_ddp_backend: str = opt("none", "if set, overrides --ddp-backend for the task", choices=TASK_DDP_BACKEND_CHOICES)
    bucket_cap_mb: int = opt(25, "bucket size for reduction")
    fix_batches_to_gpus: bool = opt(False, "don't shuffle batches between GPUs")
    find_unused_parameters: bool = opt(False, "disable unused parameter detection")
    fast_stat_sync: bool = opt(False, "[deprecated] this is now defined per criterion")
    broadcast_buffers: bool = opt(False, "copy non-trainable parameters between GPUs")
    fp16: bool = opt(False, link="common.fp16")
    memory_efficient_fp16: bool = opt(False, link="common.memory_efficient_fp16")
    bf16: bool = opt(False, link="common.bf16")
    no_reshard_after_forward: bool = opt(False, "don't reshard parameters after forward pass")
    fp32_reduce_scatter: bool = opt(False, "reduce-scatter grads in FP32")
    cpu_offload: bool = opt(False, "offload FP32 params to CPU")
    use_sharded_state: Optional[bool] = opt(False, "load and save local state dict")
    gradient_predivide_factor: Optional[float] = opt(None, "factor to predivide gradients before reduce-scatter")


@dataclass
class DatasetConfig(MetaseqDataclass):
    num_workers: int = opt(1, "how many subprocesses to use for data loading")
    num_workers_valid: int = opt(0, "how many subprocesses to use for data loading during validation")
    skip_invalid_size_inputs_valid_test: bool = opt(False, "ignore too long or too short lines in valid and test set")
    max_tokens: Optional[int] = opt(None, "maximum number of tokens in a batch")
    batch_size: Optional[int] = opt(None, "number of examples in a batch", alias="--max-sentences")
    required_batch_size_multiple: int = opt(8, "batch size will be a multiplier of this value")
    dataset_impl: Optional[str] = opt(None, "output dataset implementation", choices=DATASET_IMPL_CHOICES)
    data_buffer_size: int = opt(10, "number of batches to preload")
    skip_batches: str = opt("", "comma separated list of batch ranges to skip in multiple of num_update, e.g. "
                            "'100-200,150-250' skips updates [100,200] and [150,250]")
    train_subset: str = opt("train", "data subset to use for training (e.g. train, valid, test)")
    valid_subset: str = opt("valid", "comma separated list of data subsets to use for validation")
    combine_valid_subsets: Optional[bool] = opt(None, "comma separated list of data subsets to use for validation",
                                                alias="--combine-val")
    ignore_unused_valid_subsets: Optional[bool] = opt(False, "do not raise error if valid subsets are ignored")
    validate_interval_updates: int = opt(0, "validate every N updates")
    validate_after_updates: int = opt(0, "don't validate until reaching this many updates")
    fixed_validation_seed: Optional[int] = opt(None, "specified random seed for validation")
    disable_validation: bool = opt(False, "disable validation")
    max_tokens_valid: Optional[int] = opt(None, "maximum number of tokens in a validation batch",
                                          link="dataset.max_tokens")
    batch_size_valid: Optional[int] = opt(None, "batch size of the validation batch", link="dataset.batch_size",
                                          alias="--max-sentences-valid")
    max_valid_steps: Optional[int] = opt(None, "how many batches to evaluate", alias="--nval")
    gen_subset: str = opt("test", "data subset to generate (train, valid, test)")
    num_shards: int = opt(1, "shard generation over N shards")
    shard_id: int = opt(0, "id of the shard to generate (id < num_shards)")


@dataclass
class OptimizationConfig(MetaseqDataclass):
    max_epoch: int = opt(0, "force stop training at specified epoch")
    max_update: int = opt(0, "force stop training at specified update")
    clip_norm: float = opt(0.0, "clip threshold of gradients")
    clip_norm_type: Optional[str] = opt("l2", "either 'l2' or 'inf' to clip by l2 norm or max abs grad",
                                        choices=CLIP_GRAD_NORM_TYPE_CHOICES)
    skip_gradient_update_on_clip_norm: bool = opt(False, "skip gradient update if gnorm is higher than --clip-norm")
    ewm_ratio_to_skip_batch: float = opt(-1, "skip a batch whose loss / ewm(loss) exceeds this ratio (-1 disables)")
    update_freq: List[int] = opt(factory=lambda: [1], help="update parameters every N_i batches, when in epoch i")
    lr: List[float] = opt(factory=lambda: [0.25], help="learning rate for the first N epochs; all epochs >N use LR_N")


@dataclass
class CheckpointConfig(MetaseqDataclass):
    save_dir: str = opt("checkpoints", "path to save checkpoints")
    restore_file: str = opt("checkpoint_last.pt", "filename from which to load checkpoint")
    finetune_from_model: Optional[str] = opt(None, "finetune from a pretrained model; note that meters and lr "
                                             "scheduler will be reset")
    reset_dataloader: bool = opt(False, "if set, does not reload dataloader state from the checkpoint")
    reset_lr_scheduler: bool = opt(False, "if set, does not load lr scheduler state from the checkpoint")
    reset_meters: bool = opt(False, "if set, does not load meters from the checkpoint")
    reset_optimizer: bool = opt(False, "if set, does not load optimizer state from the checkpoint")
    optimizer_overrides: str = opt("{}", "a dictionary used to override optimizer args when loading a checkpoint")
    save_interval_epochs: int = opt(1, "save a checkpoint every N epochs")
    save_interval_updates: int = opt(0, "save a checkpoint (and validate) every N updates")
    local_save_interval_updates: int = opt(0, "save a checkpoint to local disk every N updates")
    save_last_checkpoint: bool = opt(True, "store a last checkpoint at the end of the training run")
    keep_last_epochs: int = opt(-1, "keep only the last N epoch checkpoints")
    keep_last_updates: int = opt(-1, "keep only the last N updates checkpoints")
    checkpoint_suffix: str = opt("", "suffix to add to the checkpoint file name")
    checkpoint_shard_count: int = opt(1, "number of shards containing the checkpoint")
    write_checkpoints_asynchronously: bool = opt(True, "write checkpoints asynchronously in a separate thread",
                                                 alias="--save-async")
    cloud_upload_path: Optional[str] = opt(None, "upload checkpoints asynchronously to this cloud path or nfs: dir")
    nfs_eval_script_path: Optional[str] = opt(None, "path of eval script to run on checkpoints copied to NFS")
    nfs_eval_num_attempts: int = opt(10, "number of attempts of running evals on an NFS checkpoint")
    nfs_eval_attempt_wait_minutes: int = opt(5, "time to wait between attempts of running evals")
    nfs_eval_frequency: int = opt(5000, "run evaluation only on uploaded checkpoints with multiples of this frequency")
    cluster_env: str = opt("fair", "cluster we are running on: azure/aws/fair/rsc")
    model_parallel_size: int = opt(1, link="common.model_parallel_size")
    sequence_parallel: bool = opt(False, "shard LayerNorm / residual regions along the sequence across the "
                                  "tensor-parallel group (needs --model-parallel-size > 1)")


@dataclass
class GenerationConfig(MetaseqDataclass):
    beam: int = opt(5, "beam size")
    max_len_a: float = opt(0, "generate sequences of maximum length ax + b, where x is the source length")
    max_len_b: int = opt(200, "generate sequences of maximum length ax + b, where x is the source length")
    min_len: int = opt(1, "minimum generation length")
    sampling: bool = opt(False, "sample hypotheses instead of using beam search")
    sampling_topp: float = opt(-1.0, "sample from the smallest set whose cumulative probability mass exceeds p")
    temperature: float = opt(1.0, "temperature for generation")
    no_seed_provided: bool = opt(False, "if set then no seed was provided for generation")
    buffer_size: int = opt(0, "read this many sentences into a buffer before processing them")
    input: str = opt("-", "file to read from; use - for stdin")


@dataclass
class CommonEvalConfig(MetaseqDataclass):
    path: Optional[str] = opt(None, "path(s) to model file(s), colon separated")
    quiet: bool = opt(False, "only print final scores")
    model_overrides: str = opt("{}", "a dictionary used to override model args at generation")
    results_path: Optional[str] = opt(None, "path to save eval results (optional)")


@dataclass
class ReshardConfig(MetaseqDataclass):
    save_dir: Optional[str] = opt(None, "where to save the resharded checkpoints")
    save_prefix: Optional[str] = opt("reshard", "save to <save-dir>/<save-prefix>-shard<i>.pt")
    target_world_size: Optional[int] = opt(128, "the maximum number of GPUs you want to use to evaluate")
    do_pad: Optional[bool] = opt(False, "add padding to make sure that running on target world size works")


@dataclass
class EvalLMConfig(MetaseqDataclass):
    score_sequences: bool = opt(False, "if set, uses the ScoreSequencesTask")
    output_word_probs: bool = opt(False, "if set, outputs words and their predicted log probabilities")
    output_word_stats: bool = opt(False, "if set, outputs word statistics such as word count, average probability")
    context_window: int = opt(0, "ensures that every evaluated token has access to a context of at least this size")
    softmax_batch: int = opt(sys.maxsize, "if BxT is more than this, will batch the softmax over vocab to this amount")
    max_valid_steps: Optional[int] = opt(None, "how many batches to evaluate", alias="--nval")


@dataclass
class EMAConfig(MetaseqDataclass):
    store_ema: bool = opt(False, "store exponential moving average shadow model")
    ema_decay: float = opt(0.9999, "decay for exponential moving average model")
    ema_start_update: int = opt(0, "start EMA update after this many model updates")
    ema_seed_model: Optional[str] = opt(None, "seed to load EMA model from; used to load EMA model separately")
    ema_update_freq: int = opt(1, "do EMA update every this many model updates")
    ema_fp32: bool = opt(False, "if true, store EMA model in fp32 even if model is in fp16")


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
