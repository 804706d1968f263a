"""Optimizer-state sharding across data-parallel ranks (ZeRO stage 1) for the non-FSDP backends.

The reference wraps the optimizer in fairscale's ``OSS`` (metaseq/optim/shard.py:18-57).  This module has the
same effect without the dependency: parameters are assigned to ranks greedily by size, each rank builds the
inner optimizer over its own parameters only (so it alone holds their moments), and after a step every
parameter is broadcast from its owner."""
from __future__ import annotations

from typing import Any, Dict, List

import torch
import torch.distributed as dist

from metaseq_b200.parallel import utils as dist_utils


def partition_parameters(param_groups, world_size: int) -> List[List[Dict[str, Any]]]:
    """Per rank, a list of param groups (same hyper-parameters, subset of parameters), balanced by numel."""
    loads = [0] * world_size
    per_rank = [[] for _ in range(world_size)]
    for group in param_groups:
        buckets = [[] for _ in range(world_size)]
        for p in sorted(group["params"], key=lambda t: -t.numel()):
            r = loads.index(min(loads))
            buckets[r].append(p)
            loads[r] += p.numel()
        for r in range(world_size):
            g = {k: v for k, v in group.items() if k != "params"}
            g["params"] = buckets[r]
            per_rank[r].append(g)
    return per_rank


class ShardedOptimizer(torch.optim.Optimizer):
    def __init__(self, param_groups, optim_cls, group=None, **defaults):
        self.group = group
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        all_groups = [dict(g) for g in param_groups]
        super().__init__(all_groups, defaults)
        self._partition = partition_parameters(self.param_groups, self.world_size)
        self._owner = {id(p): r for r, groups in enumerate(self._partition) for g in groups for p in g["params"]}
        mine = [g for g in self._partition[self.rank]]
        self.optim = optim_cls([g for g in mine if g["params"]] or [{"params": []}], **defaults)

    @property
    def disable_mem_eff_fp16_loading_hack(self):
        return True

    def __getattr__(self, name):
        if name.startswith("supports") and hasattr(self.__dict__.get("optim"), name):
            return getattr(self.optim, name)
        raise AttributeError("'ShardedOptimizer' object has no attribute {0!r}".format(name))

    def _sync_hyperparameters(self):
        for full, local in zip(self.param_groups, self.optim.param_groups):
            for k, v in full.items():
                if k != "params":
                    local[k] = v

    def step(self, closure=None, **kwargs):
        self._sync_hyperparameters()
        loss = self.optim.step(closure, **kwargs) if closure is not None else self.optim.step(**kwargs)
        if self.world_size > 1:
            for g in self.param_groups:
                for p in g["params"]:
                    src = dist.get_global_rank(self.group, self._owner[id(p)]) if self.group is not None \
                        else self._owner[id(p)]
                    dist.broadcast(p.data, src=src, group=self.group)
        return loss

    def state_dict(self):
        return self.optim.state_dict()

    def load_state_dict(self, state_dict):
        self.optim.load_state_dict(state_dict)

    def broadcast_global_state_dict(self, state_dict: Dict[str, Any]) -> Dict[str, Any]:
        """Sends rank 0's copy of a consolidated state dict to every rank; each rank then loads its own part."""
        return dist_utils.broadcast_object(state_dict, src_rank=0, group=self.group)


def shard_(optimizer, group):
    """Replaces ``optimizer.optimizer`` (a ``torch.optim.Optimizer`` held by a framework optimizer) in place."""
    inner = optimizer.optimizer
    optimizer.optimizer = ShardedOptimizer(inner.param_groups, type(inner), group=group, **optimizer.optimizer_config)
