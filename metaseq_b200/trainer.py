"""Training runtime: owns model, criterion, optimizer, LR scheduler and the data iterator,
runs one update per ``train_step`` and (de)serialises all of it.

Step semantics follow the reference (metaseq/trainer.py:721-968): per-update seed
``seed + num_updates``; forward/backward through ``task.train_step``; logging outputs summed
over the data-parallel group in one all-reduce; gradients multiplied by
``dp_world / sample_size`` (folded lazily into the fp16 optimizer's factor); gradient-norm
clipping with the tensor-parallel norm aggregated across ranks; ``OverflowError`` from the
loss scaler skips the update without advancing ``num_updates``; a non-finite norm outside
fp16 re-runs the step under the NaN detector and raises; loss-spike detection through an
exponentially weighted mean of the loss; LR scheduler stepped from ``set_num_updates``.

Checkpoint state layout (:352-408): ``cfg``, ``model``, ``criterion``,
``optimizer_history``, ``task_state``, ``extra_state`` (metrics, previous_training_time,
ewm_loss, train_iterator, rng_tracker_states), ``last_optimizer_state``, ``shard_metadata``.
"""
from __future__ import annotations

import contextlib
import functools
import logging
import math
import os
import sys
import time
from argparse import Namespace
from itertools import chain
from typing import Any, Dict, List, Optional

import torch

from metaseq_b200 import checkpoint_utils, models, optim, utils
from metaseq_b200.dataclass.utils import Cfg
from metaseq_b200.logging import meters, metrics
from metaseq_b200.nan_detector import NanDetector
from metaseq_b200.ops import autograd as ops_autograd
from metaseq_b200.optim import lr_scheduler
from metaseq_b200.parallel import mpu
from metaseq_b200.parallel import utils as dist_utils
from metaseq_b200.parallel.fsdp import FullyShardedDataParallel

logger = logging.getLogger(__name__)


class Trainer:
    def __init__(self, cfg, task, model, criterion):
        if isinstance(cfg, Namespace):
            from metaseq_b200.dataclass.utils import convert_namespace_to_config

            cfg = convert_namespace_to_config(cfg)
        self.cfg, self.task = cfg, task
        self.cuda = torch.cuda.is_available() and not cfg.common.cpu
        self.device = torch.device("cuda" if self.cuda else "cpu")
        # lazily built members
        self._optimizer = self._lr_scheduler = self._optim_history = None
        self._wrapped_model = self._wrapped_criterion = self._ema = None
        self._dummy_batch = None
        # progress and loss-spike bookkeeping
        self._num_updates = 0
        self._ewm_loss = None
        self._skipped_loss_spikes = 0
        self._warn_once = set()
        self._model, self._criterion = self._place(model, criterion)
        self._grad_norm_buf = None
        if self.cuda and self.data_parallel_world_size > 1:
            self._grad_norm_buf = torch.zeros(self.data_parallel_world_size, dtype=torch.double, device=self.device)
        self.cuda_env, self.cuda_env_arr = self._survey_devices()
        # wall-clock accounting (restored from checkpoints)
        metrics.log_start_time("wall", priority=790, round=2)
        self._start_time = time.time()
        self._previous_training_time = 0
        self._cumulative_training_time = None

    def _place(self, model, criterion):
        """Casts (unless the sharded wrapper owns the dtype) and moves model and criterion to the training device,
        then re-ties parameters that were shared before the move."""
        tied = _catalog_shared_params(model)
        c = self.cfg.common
        if not self.is_fsdp:
            dtype = torch.float16 if (c.fp16 or c.memory_efficient_fp16) else (torch.bfloat16 if c.bf16 else None)
            if dtype is not None:
                model, criterion = model.to(dtype=dtype), criterion.to(dtype=dtype)
        offloaded = self.is_fsdp and getattr(self.cfg.distributed_training, "cpu_offload", False)
        if not offloaded:  # offloaded shards stay in host memory; their units compute on the device by themselves
            model = model.to(device=self.device)
        criterion = criterion.to(device=self.device)
        for first, *others in tied:
            owner = _get_module_by_path(model, first)
            for path in others:
                logger.info(f"detected shared parameter: {first} <- {path}")
                _set_module_by_path(model, path, owner)
        return model, criterion

    def _survey_devices(self):
        """This rank's GPU description and every rank's (printed once by the first data-parallel rank)."""
        if not self.cuda:
            return None, None
        mine = utils.CudaEnvironment()
        everyone = [mine]
        if self.data_parallel_world_size > 1:
            everyone = dist_utils.all_gather_list(mine, group=dist_utils.get_global_group())
        if self.data_parallel_rank == 0:
            utils.CudaEnvironment.pretty_print_cuda_env_list(everyone)
        return mine, everyone

    # ------------------------------------------------------------- properties
    def reinitialize(self):
        self._lr_scheduler = None
        self._optimizer = None
        self._wrapped_criterion = None
        self._wrapped_model = None

    @property
    def data_parallel_world_size(self):
        if self.cfg.distributed_training.distributed_world_size == 1:
            return 1
        return dist_utils.get_data_parallel_world_size()

    @property
    def data_parallel_process_group(self):
        return dist_utils.get_data_parallel_group()

    @property
    def data_parallel_rank(self):
        if self.cfg.distributed_training.distributed_world_size == 1:
            return 0
        return dist_utils.get_data_parallel_rank()

    @property
    def is_data_parallel_master(self):
        return self.data_parallel_rank == 0

    @property
    def use_distributed_wrapper(self) -> bool:
        return (self.data_parallel_world_size > 1) or (self.is_fsdp and self.cfg.distributed_training.cpu_offload)

    @property
    def should_save_checkpoint_on_current_rank(self) -> bool:
        if self.is_fsdp and self.cfg.distributed_training.use_sharded_state:
            return True
        return self.is_data_parallel_master

    @property
    def checkpoint_suffix(self) -> str:
        if not self.use_sharded_state:
            return self.cfg.checkpoint.checkpoint_suffix
        if self.is_fsdp:
            return self.cfg.checkpoint.checkpoint_suffix + "-shard{0}".format(self.data_parallel_rank)
        return self.cfg.checkpoint.checkpoint_suffix or ""

    @property
    def is_fsdp(self):
        return self.cfg.distributed_training.ddp_backend == "fully_sharded"

    @property
    def use_sharded_state(self):
        return bool(self.cfg.distributed_training.use_sharded_state)

    @property
    def criterion(self):
        if self._wrapped_criterion is None:
            self._wrapped_criterion = self._criterion
        return self._wrapped_criterion

    @property
    def model(self):
        if self._wrapped_model is None:
            if self.use_distributed_wrapper and not self.is_fsdp:
                from metaseq_b200.models.distributed_model import DistributedModel

                self._wrapped_model = DistributedModel(self.cfg.distributed_training, self._model,
                                                       process_group=self.data_parallel_process_group,
                                                       device=self.device)
            else:
                self._wrapped_model = self._model
        return self._wrapped_model

    @property
    def ema(self):
        if self._ema is None:
            self._build_ema()
        return self._ema

    def _build_ema(self):
        if not getattr(self.cfg.ema, "store_ema", False):
            return
        from metaseq_b200.models.ema import build_ema

        self._ema = build_ema(self._sharded_twin() if self.is_fsdp else self._model, self.cfg.ema, self.device)
        logger.info("Exponential Moving Average Shadow Model is initialized.")

    def _sharded_twin(self):
        """A second fully sharded instance of the model holding the same state as the trained one (a sharded
        model cannot be deep-copied: its units share process groups and gathered buffers).  The shadow needs no
        gathered copies, so it uses the library collectives (metaseq/trainer.py:239-262)."""
        from metaseq_b200.parallel.fsdp import fsdp_enable_wrap, fsdp_wrap

        with fsdp_enable_wrap(self.cfg.distributed_training, use_sharded_state=self.use_sharded_state, comm="nccl"):
            twin = fsdp_wrap(self.task.build_model(self.cfg.model), process_group=self.data_parallel_process_group)
        twin = twin.to(device=self.device)
        state = self.model.state_dict()
        if not self.use_sharded_state and self.data_parallel_world_size > 1:
            state = dist_utils.broadcast_object(state, src_rank=0, group=self.data_parallel_process_group,
                                                dist_device=self.device if self.cuda else None)
        twin.load_state_dict(state)
        return twin

    @property
    def optimizer(self):
        if self._optimizer is None:
            self._build_optimizer()
        return self._optimizer

    @property
    def lr_scheduler(self):
        if self._lr_scheduler is None:
            self._build_optimizer()
        return self._lr_scheduler

    def _build_optimizer(self):
        params = list(filter(lambda p: p.requires_grad, chain(self.model.parameters(), self.criterion.parameters())))
        c = self.cfg.common
        if self.is_fsdp and (c.fp16 or c.memory_efficient_fp16):
            # sharded parameters: always the wrapper without an extra fp32 copy of its own; with
            # plain --fp16 the FSDP units themselves hold fp32 shards (mixed precision)
            allow_unsupported = not c.memory_efficient_fp16
            self._optimizer = optim.MemoryEfficientFP16Optimizer.build_optimizer(
                self.cfg, params, allow_unsupported=allow_unsupported)
        elif c.fp16 or c.bf16 or c.memory_efficient_fp16:
            if c.memory_efficient_fp16:
                self._optimizer = optim.MemoryEfficientFP16Optimizer.build_optimizer(self.cfg, params)
            else:
                self._optimizer = optim.FP16Optimizer.build_optimizer(self.cfg, params)
        else:
            self._optimizer = optim.build_optimizer(self.cfg.optimizer, params)
        self._lr_scheduler = lr_scheduler.build_lr_scheduler(self.cfg.lr_scheduler, self.optimizer)
        self._lr_scheduler.step_update(0)

    # ------------------------------------------------------------ checkpoints
    def consolidate_optimizer(self):
        """Sharded optimizer state stays sharded on disk; nothing to gather."""
        self._gathered_optim_state = None

    def state_dict(self, filename=None, training_finished=False) -> Dict[str, Any]:
        model_state = self.model.state_dict()
        optim_state = self._gathered_optim_state if getattr(self, "_gathered_optim_state", None) is not None \
            else self.optimizer.state_dict()
        state = {
            "cfg": self.cfg.to_container() if isinstance(self.cfg, Cfg) else self.cfg,
            "model": model_state,
            "criterion": self.criterion.state_dict() if utils.has_parameters(self.criterion) else None,
            "optimizer_history": (self._optim_history or []) + [{
                "criterion_name": self.criterion.__class__.__name__,
                "optimizer_name": self.optimizer.__class__.__name__,
                "lr_scheduler_state": self.lr_scheduler.state_dict(),
                "num_updates": self.get_num_updates(),
            }],
            "task_state": self.task.state_dict() if self.task is not None else {},
            "extra_state": {
                "metrics": metrics.state_dict(),
                "previous_training_time": self.cumulative_training_time(),
                "ewm_loss": self._ewm_loss,
            },
        }
        if getattr(self.cfg.ema, "store_ema", False) and self._ema is not None:
            state["extra_state"]["ema"] = self.ema.get_model().state_dict()
            if self.cfg.ema.ema_fp32:
                state["extra_state"]["ema_fp32_params"] = self.ema.fp32_params
        if not getattr(self.cfg.checkpoint, "no_save_optimizer_state", False):
            state["last_optimizer_state"] = optim_state
        if self.is_fsdp and self.use_sharded_state:
            state["shard_metadata"] = self.model.local_metadata_dict()
        return state

    def save_checkpoint(self, filename, extra_state, training_finished=False, async_callback_fn=None,
                        files_to_symlink_to=None):
        """Every rank that owns state writes its own file.  The device-to-host snapshot is taken
        here; serialisation and any post-save callback run on a background thread when
        ``--save-async`` is on."""
        if mpu.get_tensor_model_parallel_world_size() > 1:
            extra_state["rng_tracker_states"] = mpu.get_cuda_rng_tracker().get_states()
        with self._state_on_device():
            state = self.state_dict(filename, training_finished)
        state["extra_state"].update(extra_state)
        if not self.should_save_checkpoint_on_current_rank:
            return
        # copies to pinned host memory run on a side stream; the writer thread waits for them, this step does not
        if getattr(self, "_snapshot", None) is None:
            self._snapshot = checkpoint_utils.HostSnapshot()
        state = self._snapshot.take(state, cast_to_fp32=not (self.cfg.common.fp16 or self.cfg.common.bf16
                                                             or self.cfg.common.memory_efficient_fp16))
        self._snapshot_event = self._snapshot.event  # the next optimizer step must not overtake the copies
        logger.info(f"Saving checkpoint to {filename}")
        checkpoint_utils.write_checkpoint(
            state, filename, asynchronous=bool(self.cfg.checkpoint.write_checkpoints_asynchronously),
            async_callback_fn=async_callback_fn, files_to_symlink_to=files_to_symlink_to, ready=self._snapshot.ready)
        logger.info(f"Finished saving checkpoint to {filename}")

    @contextlib.contextmanager
    def _state_on_device(self):
        """While active, sharded units hand out their flat shards as device tensors (no synchronous copy)."""
        units = [m for m in self.model.modules() if isinstance(m, FullyShardedDataParallel)]
        saved = [u.state_dict_device for u in units]
        for u in units:
            u.state_dict_device = None
        try:
            yield
        finally:
            for u, dev in zip(units, saved):
                u.state_dict_device = dev

    def load_checkpoint(self, filename, reset_optimizer=False, reset_lr_scheduler=False, optimizer_overrides=None,
                        reset_meters=False):
        extra_state, self._optim_history, last_optim_state = None, [], None
        is_distributed = self.data_parallel_world_size > 1
        bexists = False
        logger.info(f"attempting to load checkpoint from: {filename}")
        if filename is not None and (os.path.isfile(filename)
                                     or checkpoint_utils.sharded_files_exist(filename, self.checkpoint_suffix)):
            bexists = True
        if bexists:
            logger.info(f"Preparing to load checkpoint {filename}")
            load_on_all_ranks = self.is_fsdp or mpu.get_tensor_model_parallel_world_size() > 1 or not is_distributed
            if load_on_all_ranks or self.is_data_parallel_master:
                state = checkpoint_utils.load_checkpoint_to_cpu(
                    filename, load_on_all_ranks=load_on_all_ranks,
                    num_shards_expected=self.data_parallel_world_size if self.is_fsdp else None,
                    shard_rank=self.data_parallel_rank if self.is_fsdp else None)
                last_optim_state = state.get("last_optimizer_state", None)
                if last_optim_state == -1:
                    master_path = filename.replace(f"-shard{self.data_parallel_rank}", "-shard0")
                    last_optim_state = torch.load(master_path, map_location="cpu", weights_only=False)["last_optimizer_state"]
            else:
                last_optim_state, state = None, None
            if is_distributed and not load_on_all_ranks:
                state = dist_utils.broadcast_object(state, src_rank=0, group=self.data_parallel_process_group,
                                                    dist_device=self.device if self.cuda else None)
                if self.data_parallel_rank > 0:
                    last_optim_state = state.get("last_optimizer_state", None)
            try:
                self.model.load_state_dict(state["model"], strict=True)
                del state["model"]
                if utils.has_parameters(self.criterion) and state.get("criterion") is not None:
                    self.criterion.load_state_dict(state["criterion"], strict=True)
            except Exception:
                raise Exception(f"Cannot load model parameters from checkpoint {filename}; please ensure that the "
                                "architectures match.")
            extra_state = state["extra_state"]
            self._optim_history = state["optimizer_history"]
        if last_optim_state is not None and not reset_optimizer:
            self._build_optimizer()
            last_optim = self._optim_history[-1]
            assert last_optim["criterion_name"] == self.criterion.__class__.__name__, \
                f"Criterion does not match; please reset the optimizer (--reset-optimizer). " \
                f"{last_optim['criterion_name']} vs {self.criterion.__class__.__name__}"
            assert last_optim["optimizer_name"] == self.optimizer.__class__.__name__, \
                f"Optimizer does not match; please reset the optimizer (--reset-optimizer). " \
                f"{last_optim['optimizer_name']} vs {self.optimizer.__class__.__name__}"
            if not reset_lr_scheduler:
                self.lr_scheduler.load_state_dict(last_optim["lr_scheduler_state"])
            self.optimizer.load_state_dict(last_optim_state, optimizer_overrides)
            self.set_num_updates(last_optim["num_updates"])
        if extra_state is not None:
            itr_state = extra_state.get("train_iterator", {})
            epoch = itr_state.get("epoch", 1)
            if "previous_training_time" in extra_state:
                self._previous_training_time = extra_state["previous_training_time"]
                self._start_time = time.time()
            if "ewm_loss" in extra_state:
                self._ewm_loss = extra_state["ewm_loss"]
            self.lr_step(epoch)
            if itr_state.get("version", 1) >= 2 and itr_state.get("iterations_in_epoch", 1) == 0:
                reset_meters = True
            if "metrics" in extra_state and not reset_meters:
                metrics.load_state_dict(extra_state["metrics"])
                for meter in metrics.get_meters("default").values():
                    if isinstance(meter, meters.TimeMeter):
                        meter.reset()
            if getattr(self.cfg.ema, "store_ema", False):
                if "ema" in extra_state:
                    self.ema.restore(extra_state["ema"], build_fp32_params=False)
                    if self.cfg.ema.ema_fp32 and "ema_fp32_params" in extra_state:
                        self.ema.build_fp32_params(extra_state["ema_fp32_params"])
                else:
                    logger.warning("EMA not found in checkpoint. But store_ema is True. EMA is re-initialized.")
                    self.ema.restore(state["model"] if "model" in state else self._model.state_dict(),
                                     build_fp32_params=self.cfg.ema.ema_fp32)
            if "rng_tracker_states" in extra_state and mpu.get_tensor_model_parallel_world_size() > 1:
                mpu.get_cuda_rng_tracker().set_states(extra_state["rng_tracker_states"])
            logger.info(f"Loaded checkpoint {filename} (epoch {epoch} @ {self.get_num_updates()} updates)")
        else:
            logger.info(f"No existing checkpoint found {filename}")
        return extra_state

    # ------------------------------------------------------------------- data
    def _batch_iterator(self, split: str, *, training: bool, epoch: int, sharded: bool, disable_iterator_cache: bool):
        """The task's batch iterator for a split, with the batching limits of training or of validation.  Its first
        batch becomes the stand-in that a rank trains on (with zero weight) when it runs out of data early."""
        d = self.cfg.dataset
        limits = [self.task.max_positions(), self.model.max_positions()] + ([d.max_tokens] if training else [])
        itr = self.task.get_batch_iterator(
            dataset=self.task.dataset(split), epoch=epoch, seed=self.cfg.common.seed,
            max_tokens=d.max_tokens if training else d.max_tokens_valid,
            max_sentences=d.batch_size if training else d.batch_size_valid,
            max_positions=utils_resolve_max_positions(*limits),
            ignore_invalid_inputs=True if training else d.skip_invalid_size_inputs_valid_test,
            required_batch_size_multiple=d.required_batch_size_multiple,
            num_shards=self.data_parallel_world_size if sharded else 1,
            shard_id=self.data_parallel_rank if sharded else 0,
            num_workers=d.num_workers if training else d.num_workers_valid,
            data_buffer_size=d.data_buffer_size, disable_iterator_cache=disable_iterator_cache,
            skip_remainder_batch=training)
        self.reset_dummy_batch(itr.first_batch)
        return itr

    def get_train_iterator(self, epoch, combine=True, load_dataset=True, data_selector=None, shard_batch_itr=True,
                           disable_iterator_cache=False):
        split = self.cfg.dataset.train_subset
        if load_dataset:
            logger.info(f"loading train data for epoch {epoch}")
            self.task.load_dataset(split, epoch=epoch, combine=combine, data_selector=data_selector)
        return self._batch_iterator(split, training=True, epoch=epoch, sharded=shard_batch_itr,
                                    disable_iterator_cache=disable_iterator_cache)

    def get_valid_iterator(self, subset, disable_iterator_cache=False):
        return self._batch_iterator(subset, training=False, epoch=1, sharded=True,
                                    disable_iterator_cache=disable_iterator_cache)

    def begin_epoch(self, epoch):
        logger.info(f"begin training epoch {epoch}")
        self.lr_step_begin_epoch(epoch)
        self.task.begin_epoch(epoch, self.get_model())

    def begin_valid_epoch(self, epoch):
        self.task.begin_valid_epoch(epoch, self.get_model())

    def reset_dummy_batch(self, batch):
        self._dummy_batch = batch

    # ------------------------------------------------------------- train step
    def start_watchdog(self):
        """Host watchdog over the training loop (``--watchdog-timeout``); returns it, or ``None`` when disabled."""
        timeout = float(getattr(self.cfg.common, "watchdog_timeout", 0.0) or 0.0)
        if timeout <= 0 or getattr(self, "watchdog", None) is not None:
            return getattr(self, "watchdog", None)
        from metaseq_b200.ops import _lib
        from metaseq_b200.utils.watchdog import StepWatchdog

        status_fn = None
        if self.device.type == "cuda" and _lib.kernels_path().exists():
            status_fn = lambda: _lib.peek_status(self.device)  # noqa: E731
        self.watchdog = StepWatchdog(timeout, status_fn=status_fn).start()
        return self.watchdog

    @metrics.aggregate("train")
    def train_step(self, samples, raise_oom=False):
        """One optimizer update over ``samples`` (a list of micro-batches)."""
        if getattr(self, "watchdog", None) is not None:
            self.watchdog.beat()
        self._set_seed()
        self.model.train()
        self.criterion.train()
        self.zero_grad()
        # the loss kernels store their gradient already multiplied by the loss scale that backward will bring
        scaler = getattr(self.optimizer, "scaler", None)
        ops_autograd.set_upstream_grad_hint(scaler.loss_scale if scaler is not None else None)
        metrics.log_start_time("train_wall", priority=800, round=2)
        logging_outputs, sample_size = [], 0
        for i, sample in enumerate(samples):
            sample, is_dummy_batch = self._prepare_sample(sample)

            def maybe_no_sync():
                if self.data_parallel_world_size > 1 and hasattr(self.model, "no_sync") and i < len(samples) - 1:
                    return self.model.no_sync()
                return contextlib.ExitStack()

            try:
                with maybe_no_sync(), self._rank_seed(self.get_num_updates()):
                    loss, sample_size_i, logging_output = self.task.train_step(
                        sample=sample, model=self.model, criterion=self.criterion, optimizer=self.optimizer,
                        update_num=self.get_num_updates(), ignore_grad=is_dummy_batch)
                    del loss
                if is_dummy_batch:
                    sample_size_i = 0 * sample_size_i if torch.is_tensor(sample_size_i) else 0
                    logging_output = {k: 0 * v for k, v in logging_output.items()}
                logging_outputs.append(logging_output)
                sample_size += sample_size_i
                if self.cuda and self.get_num_updates() == 0:
                    torch.cuda.empty_cache()
            except RuntimeError as e:
                if "out of memory" in str(e):
                    self._log_oom(e)
                    if raise_oom:
                        raise e
                raise e
        if torch.is_tensor(sample_size):
            sample_size = sample_size.float()
        else:
            sample_size = float(sample_size)
        local_sample_size = sample_size
        if self._sync_stats():
            train_time = self._local_cumulative_training_time()
            logging_outputs, (sample_size, total_train_time) = self._aggregate_logging_outputs(
                logging_outputs, sample_size, train_time)
            self._cumulative_training_time = total_train_time / self.data_parallel_world_size
        overflow = False
        logger.debug(f"[{self.get_num_updates()}] done with fwd, bwd")
        try:
            self.optimizer.all_reduce_grads(self.model)
            if utils.has_parameters(self.criterion):
                self.optimizer.all_reduce_grads(self.criterion)
            # gradients were averaged (FSDP / DDP) over the data-parallel ranks; turn that into a
            # sum divided by the global sample size
            numer = self.data_parallel_world_size if self._sync_stats() else 1
            self.optimizer.multiply_grads(numer / (float(sample_size) or 1.0))
            grad_norm = self.clip_grad_norm(self.cfg.optimization.clip_norm, self.cfg.optimization.clip_norm_type,
                                            self.cfg.optimization.skip_gradient_update_on_clip_norm)
            self._check_grad_norms(grad_norm)
            self.last_grad_norm = grad_norm
            if not torch.isfinite(torch.as_tensor(grad_norm)).all():
                raise FloatingPointError("gradients are Nan/Inf")
            # skip the update when the loss spiked against its running mean
            loss_now = sum(float(log.get("loss", 0)) for log in logging_outputs) / max(float(sample_size), 1.0) \
                / math.log(2)
            ratio = self.skip_spike(loss_now, self.cfg.optimization.ewm_ratio_to_skip_batch)
            if ratio > 1.0 and self._spike_guard_on(self.cfg.optimization.ewm_ratio_to_skip_batch):
                # a loss above its running mean damps this update by ratio^-4 (the schedule restores the rate at
                # the next update)
                new_lr = self.optimizer.get_lr() / (ratio ** 4)
                self.optimizer.set_lr(new_lr)
                logger.info(f"Scaling LR by {1.0 / ratio ** 4:.2f} to {new_lr:.6f}")
            if getattr(self, "_snapshot_event", None) is not None:
                # a checkpoint snapshot may still be reading parameters and optimizer state on its side stream
                torch.cuda.current_stream().wait_event(self._snapshot_event)
                self._snapshot_event = None
            self.task.optimizer_step(self.optimizer, model=self.model, update_num=self.get_num_updates())
            if self.is_fsdp:
                self.model.after_optimizer_step()
            logger.debug(f"[{self.get_num_updates()}] done with optimizer step")
        except FloatingPointError:
            self.zero_grad()
            with NanDetector(self.get_model()), self._rank_seed(self.get_num_updates()):
                for _, sample in enumerate(samples):
                    sample, _ = self._prepare_sample(sample)
                    self.task.train_step(sample, self.model, self.criterion, self.optimizer, self.get_num_updates(),
                                         ignore_grad=False)
            raise
        except OverflowError as e:
            overflow = True
            logger.info(f"NOTE: gradient overflow detected, ignoring gradient, {str(e)}")
            grad_norm = torch.tensor(0.0, device=self.device)
            self.zero_grad()
        except RuntimeError as e:
            if "out of memory" in str(e):
                self._log_oom(e)
                logger.error("OOM during optimization, irrecoverable")
            raise e
        logging_output = None
        if not overflow:
            self.set_num_updates(self.get_num_updates() + 1)
            if getattr(self.cfg.ema, "store_ema", False):
                self.ema.step(self.get_model(), self.get_num_updates())
                metrics.log_scalar("ema_decay", self.ema.get_decay(), priority=10000, round=5, weight=0)
            if self.cuda and self.cuda_env is not None and not getattr(self.cfg.common, "skip_gpu_mem_stats", False):
                self._log_gpu_mem_stats()
            logging_output = self._reduce_and_log_stats(logging_outputs, sample_size, grad_norm)
            if self.cuda and self.cfg.common.empty_cache_freq > 0 and (
                    (self.get_num_updates() + self.cfg.common.empty_cache_freq - 1) % self.cfg.common.empty_cache_freq == 0):
                torch.cuda.empty_cache()
        if self.cfg.common.fp16 and not self.cfg.common.bf16 and getattr(self.optimizer, "scaler", None) is not None:
            metrics.log_scalar("loss_scale", self.optimizer.scaler.loss_scale, priority=700, round=4, weight=0)
            metrics.log_scalar("scale_window", self.optimizer.scaler.scale_window, priority=700, round=4, weight=0)
        metrics.log_stop_time("train_wall")
        return logging_output

    @metrics.aggregate("valid")
    def valid_step(self, sample, num_step=0, raise_oom=False):
        with torch.no_grad():
            self.model.eval()
            self.criterion.eval()
            self.zero_grad()
            sample, is_dummy_batch = self._prepare_sample(sample)
            try:
                with self._rank_seed(num_step + self.get_num_updates()):
                    _loss, sample_size, logging_output = self.task.valid_step(sample, self.model, self.criterion)
            except RuntimeError as e:
                if "out of memory" in str(e):
                    self._log_oom(e)
                    if not raise_oom:
                        logger.warning("ran out of memory in validation step, retrying batch")
                        for p in self.model.parameters():
                            if p.grad is not None:
                                p.grad = None
                        if self.cuda:
                            torch.cuda.empty_cache()
                        return self.valid_step(sample, raise_oom=True)
                raise e
            logging_outputs = [logging_output]
            if is_dummy_batch:
                sample_size = sample_size * 0
        if self.data_parallel_world_size > 1:
            logging_outputs, (sample_size,) = self._aggregate_logging_outputs(logging_outputs, sample_size)
        return self._reduce_and_log_stats(logging_outputs, sample_size)

    def _rank_seed(self, update: int):
        """``--seed-per-rank``: inside the block every rank draws from its own stream, seeded from (seed, update,
        rank); the generators are put back afterwards.  Without the flag: nothing."""
        if getattr(self.cfg.common, "seed_per_rank", False):
            return utils.set_rank_seed(self.cfg.common.seed, update)
        return contextlib.nullcontext()

    def zero_grad(self):
        self.optimizer.zero_grad()
        if self.is_fsdp and isinstance(self.model, FullyShardedDataParallel):
            self.model.zero_grad()

    # ------------------------------------------------------------ lr / updates
    def _publish_lr(self, value):
        """Logs what the schedule returned (one number, or one per parameter group) and gives back the headline
        value."""
        if not isinstance(value, dict):
            metrics.log_scalar("lr", value, weight=0, priority=300)
            return value
        for group, lr in value.items():
            metrics.log_scalar(f"lr_{group}", lr, weight=0, priority=300)
        return value["default"] if "default" in value else next(iter(value.values()))

    def lr_step_update(self):
        """Moves the schedule to the current update count."""
        return self._publish_lr(self.lr_scheduler.step_update(self._num_updates))

    def lr_step_begin_epoch(self, epoch):
        self.lr_scheduler.step_begin_epoch(epoch)
        return self.lr_step_update()

    def lr_step(self, epoch, val_loss=None):
        """End of an epoch (and of its validation)."""
        self.lr_scheduler.step(epoch, val_loss)
        return self.lr_step_update()

    def get_num_updates(self):
        return self._num_updates

    def set_num_updates(self, num_updates):
        self._num_updates = num_updates
        self.lr_step_update()
        metrics.log_scalar("num_updates", num_updates, weight=0, priority=200)

    def get_lr(self):
        return self.optimizer.get_lr()

    def get_meter(self, name):
        return metrics.get_meter("train", name)

    def get_model(self):
        """The model without its data-parallel wrapper."""
        return self._model

    def get_criterion(self):
        return self._criterion

    def clip_grad_norm(self, clip_norm, clip_norm_type="l2", skip_gradient_update_on_clip_norm=False):
        if self.optimizer.__class__.__name__ in ("MemoryEfficientFP16Optimizer", "FP16Optimizer"):
            return self.optimizer.clip_grad_norm(
                clip_norm, clip_norm_type, aggregate_norm_fn=self._aggregate_model_parallel_grad_norm,
                skip_gradient_update_on_clip_norm=skip_gradient_update_on_clip_norm)
        return self.optimizer.clip_grad_norm(clip_norm, clip_norm_type,
                                             aggregate_norm_fn=self._aggregate_model_parallel_grad_norm)

    def _aggregate_model_parallel_grad_norm(self, norm_type_or_total, total_norm=None):
        """Combines the gradient norm across tensor-parallel ranks (each holds different slices of
        the parallel weights; replicated parameters are counted once per rank, as in the reference)."""
        if total_norm is None:
            total_norm, norm_type = norm_type_or_total, self.cfg.optimization.clip_norm_type
        else:
            norm_type = norm_type_or_total
        if mpu.get_tensor_model_parallel_world_size() == 1:
            return total_norm
        out = total_norm.clone()
        if norm_type == "inf":
            dist_utils.all_reduce(out, group=dist_utils.get_model_parallel_group(), op="max")
        else:
            out = out ** 2
            dist_utils.all_reduce(out, group=dist_utils.get_model_parallel_group())
            out = out ** 0.5
        return out

    @staticmethod
    def _spike_guard_on(threshold) -> bool:
        return threshold is not None and threshold > 0

    def skip_spike(self, loss_now: float, ewm_ratio_to_skip_batch: float, span: int = 9) -> float:
        """Ratio of the current loss (base 2) to its exponentially weighted mean, returned every step.  With the
        guard on (a positive threshold) a loss above ``threshold x mean`` counts as a spike and leaves the mean
        untouched, so one bad batch does not raise the baseline it is compared with
        (metaseq/trainer.py:1115-1141); with the guard off the mean follows every step and is only logged."""
        if self._ewm_loss is None or not math.isfinite(self._ewm_loss):
            self._ewm_loss = loss_now
        mean = self._ewm_loss
        ratio = loss_now / mean if mean > 0 else 1.0
        if self._spike_guard_on(ewm_ratio_to_skip_batch) and ratio > ewm_ratio_to_skip_batch:
            self._skipped_loss_spikes += 1
            metrics.log_scalar("skipped_loss_spikes", self._skipped_loss_spikes, priority=720, round=0, weight=0)
        else:
            alpha = 2.0 / (span + 1)
            self._ewm_loss = (1 - alpha) * mean + alpha * loss_now
        metrics.log_scalar("ewm_loss", self._ewm_loss, priority=700, round=2, weight=0)
        metrics.log_scalar("ewm_loss_ratio", ratio, priority=710, round=4, weight=0)
        return ratio

    def cumulative_training_time(self):
        if self._cumulative_training_time is None:
            return self._local_cumulative_training_time()
        return self._cumulative_training_time

    def _local_cumulative_training_time(self):
        return time.time() - self._start_time + self._previous_training_time

    # ---------------------------------------------------------------- samples
    def _prepare_sample(self, sample, is_dummy=False):
        if sample == "DUMMY":
            raise Exception("Trying to use an uninitialized 'dummy' batch. This usually indicates that the total "
                            "number of batches is smaller than the number of participating GPUs. Try reducing the "
                            "batch size or using fewer GPUs.")
        if sample is None or len(sample) == 0:
            assert self._dummy_batch is not None and len(self._dummy_batch) > 0, f"Invalid dummy batch: {self._dummy_batch}"
            sample, _ = self._prepare_sample(self._dummy_batch, is_dummy=True)
            return sample, True
        if self.cuda:
            sample = utils.move_to_cuda(sample)
        return sample, is_dummy

    def _set_seed(self):
        utils.set_torch_seed(self.cfg.common.seed + self.get_num_updates())

    def _sync_stats(self):
        if self.data_parallel_world_size == 1:
            return False
        return True

    def _log_oom(self, exc):
        logger.warning(f"OOM: Ran out of memory with exception: {exc}")
        if torch.cuda.is_available() and hasattr(torch.cuda, "memory_summary"):
            for idx in range(torch.cuda.device_count()):
                logger.warning(torch.cuda.memory_summary(device=idx))
        sys.stderr.flush()

    def _aggregate_logging_outputs(self, logging_outputs: List[Dict[str, Any]], *extra_stats_to_sum):
        if self.task.__class__.logging_outputs_can_be_summed(self.get_criterion()):
            return self._fast_stat_sync_sum(logging_outputs, *extra_stats_to_sum)
        return self._all_gather_list_sync(logging_outputs, *extra_stats_to_sum)

    def _all_gather_list_sync(self, logging_outputs, *extra_stats_to_sum):
        results = list(zip(*dist_utils.all_gather_list(
            [logging_outputs] + list(extra_stats_to_sum),
            max_size=getattr(self.cfg.common, "all_gather_list_size", 16384),
            group=self.data_parallel_process_group)))
        logging_outputs, extra = results[0], results[1:]
        logging_outputs = list(chain.from_iterable(logging_outputs))
        return logging_outputs, [sum(s) for s in extra]

    def _fast_stat_sync_sum(self, logging_outputs, *extra_stats_to_sum):
        data = {}
        for i, stat in enumerate(extra_stats_to_sum):
            data["extra_stats_" + str(i)] = stat
        if len(logging_outputs) > 0:
            for k in list(logging_outputs[0].keys()):
                v = sum(log[k] for log in logging_outputs if k in log)
                data["logging_outputs_" + k] = v
        data = dist_utils.all_reduce_dict(data, device=self.device, group=self.data_parallel_process_group)
        extra = [data["extra_stats_" + str(i)] for i in range(len(extra_stats_to_sum))]
        if len(logging_outputs) > 0:
            logging_outputs = [{k: data["logging_outputs_" + k] for k in logging_outputs[0].keys()}]
        else:
            logging_outputs = []
        return logging_outputs, extra

    def _check_grad_norms(self, grad_norm):
        """All data-parallel ranks must see the same gradient norm; a mismatch means the ranks have
        diverged (different data ordering or non-deterministic kernels feeding a collective)."""
        if self._grad_norm_buf is None:
            return
        self._grad_norm_buf.zero_()
        self._grad_norm_buf[self.data_parallel_rank] = float(grad_norm)
        dist_utils.all_reduce(self._grad_norm_buf, group=self.data_parallel_process_group)

        def is_consistent(t):
            max_abs_diff = torch.max(torch.abs(t - t[0]))
            return (not torch.isfinite(t).any()) or bool((max_abs_diff / (t[0] + 1e-6) < 1e-6).all())

        if not is_consistent(self._grad_norm_buf):
            pretty = "\n".join("rank {:3d} = {:.8f}".format(r, n) for r, n in enumerate(self._grad_norm_buf.tolist()))
            raise FloatingPointError(
                "Fatal error: gradients are inconsistent between workers. Try --ddp-backend=legacy_ddp. "
                "Or are you mixing up different generation of GPUs in training?\n" + "-" * 80
                + "\n{}\n".format(pretty) + "-" * 80)

    def _reduce_and_log_stats(self, logging_outputs, sample_size, grad_norm=None):
        if grad_norm is not None and (not torch.is_tensor(grad_norm) or torch.isfinite(grad_norm)):
            metrics.log_speed("ups", 1.0, priority=100, round=2)
            metrics.log_scalar("gnorm", grad_norm, priority=400, round=3)
            if self.cfg.optimization.clip_norm > 0:
                gn = float(grad_norm)
                metrics.log_scalar("clip", 100.0 if gn > self.cfg.optimization.clip_norm else 0.0, priority=500, round=1)
            if self.is_fsdp and not getattr(self.cfg.common, "quiet_logs", False) and \
                    getattr(self.cfg.common, "log_param_stats", False):
                self._log_param_stats()
        with metrics.aggregate() as agg:
            if logging_outputs is not None:
                self.task.reduce_metrics(logging_outputs, self.get_criterion())
                del logging_outputs
            if "loss" not in agg:
                if "loss" not in self._warn_once:
                    self._warn_once.add("loss")
                    logger.warning("Criterion.reduce_metrics did not log a 'loss' value, which may break some "
                                   "functionality")
                metrics.log_scalar("loss", -1)
            logging_output = agg.get_smoothed_values()
            logging_output["sample_size"] = sample_size
            return logging_output

    def _log_param_stats(self):
        """Per flat parameter: L2 norm, maximum and the share of (near-)zero entries, of the gradient as the
        optimizer will apply it and of the parameter itself (metaseq/trainer.py:1360-1390).  The values stay on
        the device until the meters are printed."""
        factor = getattr(self.optimizer, "_multiply_factor", None)
        for name, p in self.model.named_parameters():
            if p.grad is None:
                continue
            short = name.replace(".flat_param", "").replace("module.", "").replace("decoder.layers.", "layer")
            tiny = 2 * torch.finfo(p.grad.dtype).tiny
            with torch.no_grad():
                for tag, t, prio in (("g", p.grad if factor is None else p.grad * factor, 10), ("p", p.detach(), 13)):
                    metrics.log_scalar(f"{tag}norm_{short}", t.float().norm(), priority=prio, round=4)
                    metrics.log_scalar(f"{tag}max_{short}", t.max().float(), priority=prio + 1, round=4)
                    metrics.log_scalar(f"{tag}zero_{short}", (t.abs() < tiny).float().mean(), priority=prio + 2, round=4)

    def _log_gpu_mem_stats(self):
        gb = 1024.0 ** 3
        alloc = torch.cuda.max_memory_allocated() / gb
        torch.cuda.reset_peak_memory_stats()  # the logged value is the peak of this update alone
        self.peak_gb_allocated = max(getattr(self, "peak_gb_allocated", 0.0), alloc)  # peak over all updates
        reserved = torch.cuda.max_memory_reserved() / gb
        total = self.cuda_env.total_memory_in_GB
        metrics.log_scalar("cuda_gb_allocated", alloc, priority=1500, round=1, weight=0)
        metrics.log_scalar("cuda_gb_reserved", reserved, priority=1500, round=1, weight=0)
        metrics.log_scalar("cuda_gb_free", total - alloc, priority=1500, round=1, weight=0)
        if getattr(self.cfg.common, "log_nvidia_smi", False):
            for k, v in metrics.nvidia_smi_gpu_memory_stats().items():
                metrics.log_scalar(k, v, priority=1500, round=1, weight=0)


class SpikeError(Exception):
    """A loss far above its running mean.  ``Trainer.skip_spike`` handles spikes by skipping the batch; this type is
    for callers that prefer to stop (the reference declares it without raising it: metaseq/trainer.py:1496)."""


def utils_resolve_max_positions(*args):
    """Smallest of the given limits (None entries ignored)."""
    vals = []
    for a in args:
        if a is None:
            continue
        if isinstance(a, (tuple, list)):
            vals.extend(x for x in a if x is not None)
        else:
            vals.append(a)
    return min(vals) if vals else None


def _catalog_shared_params(module, memo=None, prefix=""):
    if memo is None:
        first_call = True
        memo = {}
    else:
        first_call = False
    for name, param in module._parameters.items():
        if param is None:
            continue
        param_prefix = prefix + ("." if prefix else "") + name
        memo.setdefault(param, []).append(param_prefix)
    for name, m in module._modules.items():
        if m is None:
            continue
        sub = prefix + ("." if prefix else "") + name
        _catalog_shared_params(m, memo, sub)
    if first_call:
        return [x for x in memo.values() if len(x) > 1]


def _get_module_by_path(module, path):
    for name in path.split("."):
        module = getattr(module, name)
    return module


def _set_module_by_path(module, path, value):
    parts = path.split(".")
    for name in parts[:-1]:
        module = getattr(module, name)
    setattr(module, parts[-1], value)
