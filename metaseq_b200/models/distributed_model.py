"""Data-parallel wrapping for the non-sharded backends: torch DDP behind a proxy that keeps the
wrapped model's attributes reachable; FSDP models pass through (reference:
metaseq/models/distributed_model.py:25-74)."""
from __future__ import annotations

import logging

import torch
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel

from metaseq_b200.parallel.fsdp import FullyShardedDataParallel
from metaseq_b200.parallel.module_proxy_wrapper import ModuleProxyWrapper

logger = logging.getLogger(__name__)


def DistributedModel(cfg_dist, model, process_group, device):
    assert isinstance(model, nn.Module)
    backend = cfg_dist.ddp_backend
    if backend in ("c10d", "pytorch_ddp"):
        kwargs = dict(module=model.to(device), broadcast_buffers=cfg_dist.broadcast_buffers,
                      bucket_cap_mb=cfg_dist.bucket_cap_mb, process_group=process_group,
                      find_unused_parameters=cfg_dist.find_unused_parameters)
        if device.type == "cuda":
            kwargs.update(device_ids=[cfg_dist.device_id], output_device=cfg_dist.device_id)
        wrapped = DistributedDataParallel(**kwargs)
        return ModuleProxyWrapper(wrapped)
    if backend == "fully_sharded":
        assert isinstance(model, FullyShardedDataParallel), "expected model to already be wrapped in FSDP"
        if cfg_dist.memory_efficient_fp16:
            model = model.half()
        if not cfg_dist.cpu_offload:
            model = model.to(device=device)
        return model
    raise ValueError("Unknown --ddp-backend: " + backend)
