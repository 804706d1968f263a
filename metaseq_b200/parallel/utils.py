"""Distributed runtime: process launch, initialisation, group getters and the
control-plane collectives.

One process per GPU.  ``call_main`` either adopts the environment of an external
launcher (torchrun / SLURM: RANK, LOCAL_RANK, WORLD_SIZE, MASTER_ADDR/PORT) or
spawns ``world_size - 1`` children and runs rank 0 inline, as the reference does
(metaseq/distributed/utils.py:37-118 init-method inference, :120-193
``distributed_init``, :195-285 launch, :343-389 group getters, :392-645
collectives).  Hot-path collectives do not go through this module: they are
fused into kernels (``metaseq_b200.parallel.symm``); everything here is small,
latency-insensitive traffic on NCCL (or gloo on CPU).
"""
from __future__ import annotations

import io
import logging
import os
import pickle
import random
import signal
import socket
import struct
import subprocess
from argparse import Namespace
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional

import torch
import torch.distributed as dist

from . import mpu

logger = logging.getLogger(__name__)

_USE_MEGATRON = False
_GLOBAL_GROUP = None


def is_master(cfg_dist) -> bool:
    return getattr(cfg_dist, "distributed_rank", 0) == 0


def is_initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


# ----------------------------------------------------------- init method
def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def infer_init_method(cfg_dist, force_distributed: bool = False):
    """Fills ``distributed_init_method`` / rank / world size from the environment."""
    if getattr(cfg_dist, "distributed_init_method", None) is not None:
        return
    if all(k in os.environ for k in ("MASTER_ADDR", "MASTER_PORT", "WORLD_SIZE", "RANK")):
        # launched by torchrun / torch.distributed.run
        cfg_dist.distributed_init_method = "env://"
        cfg_dist.distributed_world_size = int(os.environ["WORLD_SIZE"])
        cfg_dist.distributed_rank = int(os.environ["RANK"])
        cfg_dist.device_id = int(os.environ.get("LOCAL_RANK", 0))
        cfg_dist.distributed_no_spawn = True
        return
    if getattr(cfg_dist, "distributed_port", -1) > 0 and "SLURM_NODELIST" in os.environ:
        _infer_slurm_init(cfg_dist)
        return
    if getattr(cfg_dist, "distributed_world_size", 1) > 1 or force_distributed:
        port = _free_port()
        cfg_dist.distributed_init_method = f"tcp://127.0.0.1:{port}"


def _infer_slurm_init(cfg_dist):
    node_list = os.environ.get("SLURM_STEP_NODELIST") or os.environ.get("SLURM_JOB_NODELIST")
    if node_list is None:
        return
    try:
        hostnames = subprocess.check_output(["scontrol", "show", "hostnames", node_list])
        host = hostnames.split()[0].decode("utf-8")
    except (subprocess.CalledProcessError, FileNotFoundError):
        return
    cfg_dist.distributed_init_method = f"tcp://{host}:{cfg_dist.distributed_port}"
    nnodes = int(os.environ.get("SLURM_NNODES", 1))
    ntasks_per_node = os.environ.get("SLURM_NTASKS_PER_NODE")
    if ntasks_per_node is None:
        ntasks_per_node = int(os.environ.get("SLURM_NTASKS", 1)) // nnodes
    ntasks_per_node = int(ntasks_per_node)
    if ntasks_per_node == 1:
        gpus_per_node = max(1, torch.cuda.device_count())
        node_id = int(os.environ.get("SLURM_NODEID", 0))
        cfg_dist.distributed_rank = node_id * gpus_per_node
        cfg_dist.distributed_world_size = nnodes * gpus_per_node
    else:
        cfg_dist.distributed_no_spawn = True
        cfg_dist.distributed_rank = int(os.environ.get("SLURM_PROCID", 0))
        cfg_dist.device_id = int(os.environ.get("SLURM_LOCALID", 0))


# --------------------------------------------------------------- init
def distributed_init(cfg) -> int:
    """Creates the default process group, the data / tensor parallel groups and seeds the
    tensor-parallel RNG tracker.  Returns this process's global rank."""
    global _USE_MEGATRON, _GLOBAL_GROUP
    d = cfg.distributed_training
    common = cfg.common
    use_cuda = torch.cuda.is_available() and not getattr(common, "cpu", False)
    backend = d.distributed_backend if use_cuda else "gloo"
    if is_initialized():
        logger.warning("Distributed is already initialized, cannot initialize twice!")
    else:
        logger.debug(f"distributed init (rank {d.distributed_rank}): {d.distributed_init_method}")
        kwargs = {}
        if use_cuda:
            try:
                kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
            except Exception:
                kwargs = {}
        dist.init_process_group(
            backend=backend,
            init_method=d.distributed_init_method,
            world_size=d.distributed_world_size,
            rank=d.distributed_rank,
            **kwargs,
        )
        logger.info(f"initialized host {socket.gethostname()} as rank {d.distributed_rank}")
        # one tiny all-reduce brings up the communicator before the first real collective
        t = torch.zeros(1, device="cuda" if use_cuda else "cpu")
        dist.all_reduce(t)
    d.distributed_rank = dist.get_rank()
    if not is_master(d):
        logging.getLogger().setLevel(logging.WARNING)
    mp_size = int(getattr(common, "model_parallel_size", 1))
    mpu.initialize_model_parallel(mp_size)
    _USE_MEGATRON = True
    mpu.model_parallel_cuda_manual_seed(int(common.seed))
    suffix = getattr(cfg.checkpoint, "checkpoint_suffix", "")
    cfg.checkpoint.checkpoint_suffix = suffix + "-model_part-{0}".format(mpu.get_tensor_model_parallel_rank())
    return d.distributed_rank


def distributed_main(i, main, cfg, kwargs):
    d = cfg.distributed_training
    if not getattr(d, "distributed_no_spawn", False):
        d.device_id = i
    use_cuda = torch.cuda.is_available() and not getattr(cfg.common, "cpu", False)
    if use_cuda:
        torch.cuda.set_device(d.device_id % max(1, torch.cuda.device_count()))
    if d.distributed_rank is None:
        d.distributed_rank = kwargs.pop("start_rank", 0) + i
    elif not getattr(d, "distributed_no_spawn", False):
        d.distributed_rank = kwargs.pop("start_rank", 0) + i
    kwargs.pop("start_rank", None)
    d.distributed_rank = distributed_init(cfg)
    after = kwargs.pop("after_distributed_init_fn", None)
    if after:
        cfg = after(cfg)
    ret = main(cfg, **kwargs)
    if is_initialized():
        dist.barrier(get_global_group())
    return ret


def _spawn_entry(i, main, cfg, kwargs):
    distributed_main(i + 1, main, cfg, kwargs)


def call_main(cfg, main, **kwargs):
    """Runs ``main(cfg, **kwargs)`` on every rank of the job and returns rank 0's result."""
    d = cfg.distributed_training
    if d.distributed_init_method is None:
        infer_init_method(d)
    if d.distributed_init_method is not None:
        if not d.distributed_no_spawn:
            start_rank = d.distributed_rank or 0
            d.distributed_rank = None
            kwargs["start_rank"] = start_rank
            n_local = min(max(1, torch.cuda.device_count()) if torch.cuda.is_available() else d.distributed_world_size,
                          d.distributed_world_size)
            return _spawn_helper(main, cfg, kwargs, n_local)
        return distributed_main(d.device_id, main, cfg, kwargs)
    # single process, single device
    if torch.cuda.is_available() and not getattr(cfg.common, "cpu", False):
        torch.cuda.set_device(d.device_id)
    return main(cfg, **kwargs)


def _spawn_helper(main, cfg, kwargs, nprocs):
    """Children get local ranks 1..n-1; rank 0 runs in this process so that its return value
    and exceptions surface directly.  Children are killed if rank 0 fails."""
    import torch.multiprocessing as mp

    ctx = None
    if nprocs > 1:
        ctx = mp.start_processes(_spawn_entry, args=(main, cfg, dict(kwargs)), nprocs=nprocs - 1, join=False,
                                 start_method="spawn")
    try:
        ret = distributed_main(0, main, cfg, kwargs)
        if ctx is not None:
            ctx.join(timeout=120)
        return ret
    except (KeyboardInterrupt, Exception):
        if ctx is not None:
            for p in ctx.processes:
                if p.is_alive():
                    os.kill(p.pid, signal.SIGKILL)
        raise


# ------------------------------------------------------------ group getters
def new_groups(grouped_ranks: List[List[int]]):
    groups = [dist.new_group(g) for g in grouped_ranks]
    my = [i for i, g in enumerate(grouped_ranks) if dist.get_rank() in g]
    return groups[my[0]]


def get_global_group():
    """A clone of WORLD used for control traffic so it never interleaves with collectives
    other components issue on the default group."""
    global _GLOBAL_GROUP
    if not is_initialized():
        return None
    if _GLOBAL_GROUP is None:
        _GLOBAL_GROUP = dist.new_group()
    return _GLOBAL_GROUP


def get_global_rank() -> int:
    return dist.get_rank() if is_initialized() else 0


def get_global_world_size() -> int:
    return dist.get_world_size() if is_initialized() else 1


def get_data_parallel_group():
    if _USE_MEGATRON and mpu.model_parallel_is_initialized():
        return mpu.get_data_parallel_group()
    return get_global_group()


def get_data_parallel_rank() -> int:
    return mpu.get_data_parallel_rank() if mpu.model_parallel_is_initialized() else get_global_rank()


def get_data_parallel_world_size() -> int:
    return mpu.get_data_parallel_world_size() if mpu.model_parallel_is_initialized() else get_global_world_size()


def get_model_parallel_group():
    return mpu.get_tensor_model_parallel_group() if mpu.model_parallel_is_initialized() else None


def get_model_parallel_rank() -> int:
    return mpu.get_tensor_model_parallel_rank()


def get_model_parallel_world_size() -> int:
    return mpu.get_tensor_model_parallel_world_size()


def get_rank(group) -> int:
    return dist.get_rank(group=group) if is_initialized() else 0


def get_world_size(group) -> int:
    return dist.get_world_size(group=group) if is_initialized() else 1


# -------------------------------------------------------------- collectives
def global_barrier():
    """Waits for every process of the job, whatever groups it belongs to (metaseq/distributed/utils.py:223)."""
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        torch.distributed.barrier(get_global_group())


def all_reduce(tensor, group=None, op="sum"):
    if not is_initialized() or get_world_size(group) == 1:
        return tensor
    rop = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op]
    dist.all_reduce(tensor, op=rop, group=group)
    return tensor


def broadcast(tensor, src, group=None):
    if is_initialized() and get_world_size(group) > 1:
        dist.broadcast(tensor, src=src, group=group)
    return tensor


def all_gather(tensor, group=None, return_tensor: bool = False):
    world = get_world_size(group)
    if world == 1:
        return tensor.unsqueeze(0) if return_tensor else [tensor]
    outs = [torch.empty_like(tensor) for _ in range(world)]
    dist.all_gather(outs, tensor.contiguous(), group=group)
    return torch.stack(outs, dim=0) if return_tensor else outs


def all_to_all(tensor, group=None):
    world = get_world_size(group)
    if world == 1:
        return tensor
    out = torch.empty_like(tensor)
    dist.all_to_all_single(out, tensor.contiguous(), group=group)
    return out


def _comm_device(group=None):
    if is_initialized() and dist.get_backend(group) == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def all_gather_list(data, group=None, max_size: int = 16384):
    """Gathers arbitrary picklable objects from every rank.  Each rank writes a
    length-prefixed pickle into its slot of a zeroed byte buffer and one SUM all-reduce
    merges the slots (same wire format idea as metaseq/distributed/utils.py:431-501)."""
    if not is_initialized() or get_world_size(group) == 1:
        return [data]
    rank, world = get_rank(group), get_world_size(group)
    enc = pickle.dumps(data)
    header = 4
    size = header + len(enc)
    if size > max_size:
        raise ValueError(f"encoded data size ({size}) exceeds max_size ({max_size})")
    dev = _comm_device(group)
    buf = torch.zeros(max_size * world, dtype=torch.uint8)
    start = rank * max_size
    buf[start:start + size] = torch.frombuffer(bytearray(struct.pack(">I", len(enc)) + enc), dtype=torch.uint8)
    buf = buf.to(dev)
    dist.all_reduce(buf, group=group)
    buf = buf.cpu()
    out = []
    try:
        for i in range(world):
            chunk = buf[i * max_size:(i + 1) * max_size]
            (n,) = struct.unpack(">I", bytes(chunk[:header].tolist()))
            if n > 0:
                out.append(pickle.loads(bytes(chunk[header:header + n].tolist())))
        return out
    except pickle.UnpicklingError:
        raise Exception(
            "Unable to unpickle data from other workers. all_gather_list requires all workers to enter the "
            "function together, so this error usually indicates that the workers have fallen out of sync."
        )


def all_reduce_dict(data: Mapping[str, Any], device, group=None) -> Dict[str, Any]:
    """Sums a dict of scalars across ranks with one all-reduce of concatenated doubles."""
    keys = list(data.keys())
    if not is_initialized() or get_world_size(group) == 1 or not keys:
        return OrderedDict((k, data[k]) for k in keys)
    comm_dev = _comm_device(group)
    vals = []
    for k in keys:
        v = data[k]
        vals.append(v.detach().to(dtype=torch.double, device=comm_dev).reshape(-1)[0:1]
                    if torch.is_tensor(v) else torch.tensor([float(v)], dtype=torch.double, device=comm_dev))
    buf = torch.cat(vals)
    dist.all_reduce(buf, group=group)
    buf = buf.to(device) if device is not None else buf
    return OrderedDict((k, buf[i]) for i, k in enumerate(keys))


def broadcast_tensors(tensors: Optional[List[torch.Tensor]], src_rank: int, group=None, dist_device=None):
    if dist_device is None:
        dist_device = _comm_device(group)
    is_src = get_rank(group) == src_rank if group is not None else get_global_rank() == src_rank
    meta = [{"size": t.size(), "dtype": t.dtype, "device": t.device} for t in tensors] if is_src else None
    meta = _broadcast_object_slow(meta, src_rank, group, dist_device)
    out = []
    for i, m in enumerate(meta):
        if is_src:
            t = tensors[i].to(dist_device)
        else:
            t = torch.zeros(m["size"], dtype=m["dtype"], device=dist_device)
        broadcast(t, src=src_rank, group=group)
        out.append(t.to(m["device"]) if m["device"].type == "cpu" else t)
    return out


@dataclass(frozen=True)
class _TensorPlaceholder:
    index: int


def _split_tensors(obj, tensors):
    if torch.is_tensor(obj):
        tensors.append(obj)
        return _TensorPlaceholder(len(tensors) - 1)
    if isinstance(obj, dict):
        return {k: _split_tensors(v, tensors) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_split_tensors(v, tensors) for v in obj]
    if isinstance(obj, tuple):
        return tuple(_split_tensors(v, tensors) for v in obj)
    return obj


def _join_tensors(obj, tensors):
    if isinstance(obj, _TensorPlaceholder):
        return tensors[obj.index]
    if isinstance(obj, dict):
        return {k: _join_tensors(v, tensors) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_join_tensors(v, tensors) for v in obj]
    if isinstance(obj, tuple):
        return tuple(_join_tensors(v, tensors) for v in obj)
    return obj


def broadcast_object(obj, src_rank: int, group=None, dist_device=None):
    """Broadcasts an arbitrary object; tensors inside travel as tensors, the rest pickled."""
    if not is_initialized() or get_world_size(group) == 1:
        return obj
    if dist_device is None:
        dist_device = _comm_device(group)
    if get_global_rank() == src_rank:
        tensors: List[torch.Tensor] = []
        skeleton = _split_tensors(obj, tensors)
        skeleton = _broadcast_object_slow(skeleton, src_rank, group, dist_device)
        tensors = broadcast_tensors(tensors, src_rank, group, dist_device)
    else:
        skeleton = _broadcast_object_slow(None, src_rank, group, dist_device)
        tensors = broadcast_tensors(None, src_rank, group, dist_device)
    return _join_tensors(skeleton, tensors)


def _broadcast_object_slow(obj, src_rank, group, dist_device):
    if get_global_rank() == src_rank:
        buffer = io.BytesIO()
        torch.save(obj, buffer)
        data = torch.frombuffer(bytearray(buffer.getvalue()), dtype=torch.uint8).to(dist_device)
        length = torch.tensor([data.numel()], dtype=torch.long, device=dist_device)
        broadcast(length, src=src_rank, group=group)
        broadcast(data, src=src_rank, group=group)
        return obj
    length = torch.zeros(1, dtype=torch.long, device=dist_device)
    broadcast(length, src=src_rank, group=group)
    data = torch.zeros(int(length.item()), dtype=torch.uint8, device=dist_device)
    broadcast(data, src=src_rank, group=group)
    return torch.load(io.BytesIO(data.cpu().numpy().tobytes()), map_location="cpu", weights_only=False)
