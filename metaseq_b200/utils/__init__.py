"""Small helpers shared across the package: sample movement, positions, seeding,
gradient norms, initialisers, dtype checks.  Behavioural reference:
metaseq/utils.py (make_positions :83-93, clip_grad_norm_ :133-229, seeds
:372-410, CudaEnvironment :413-439, init functions :508-538)."""
from __future__ import annotations

import builtins
import contextlib
import copy
import importlib
import itertools
import sys
import logging
import math
import os
import random
import re
from typing import Callable, Dict, List, Optional

import numpy as np
import torch
import torch.nn.functional as F

logger = logging.getLogger(__name__)


# ----------------------------------------------------------------- samples
def apply_to_sample(f: Callable, sample):
    if hasattr(sample, "__len__") and len(sample) == 0:
        return {}

    def _apply(x):
        if torch.is_tensor(x):
            return f(x)
        if isinstance(x, dict):
            return {k: _apply(v) for k, v in x.items()}
        if isinstance(x, list):
            return [_apply(v) for v in x]
        if isinstance(x, tuple):
            return tuple(_apply(v) for v in x)
        if isinstance(x, set):
            return {_apply(v) for v in x}
        return x

    return _apply(sample)


def move_to_cuda(sample, device=None):
    device = device or torch.cuda.current_device()
    return apply_to_sample(lambda t: t.to(device=device, non_blocking=True), sample)


def move_to_cpu(sample, cast_to_fp32: bool = True):
    def _cpu(t):
        if cast_to_fp32 and t.dtype in (torch.bfloat16, torch.float16):
            return t.to(dtype=torch.float32, device="cpu")
        return t.cpu()

    return apply_to_sample(_cpu, sample)


def item(x):
    if hasattr(x, "item"):
        return x.item()
    if hasattr(x, "__getitem__"):
        return x[0]
    return x


# --------------------------------------------------------------- positions
def make_positions(tokens: torch.Tensor, padding_idx: int) -> torch.Tensor:
    """Position of the k-th non-pad token (1-based k) is ``k + padding_idx``; pads map to
    ``padding_idx``.  With OPT's ``padding_idx = 1`` the first real token gets index 2."""
    mask = tokens.ne(padding_idx).int()
    return (torch.cumsum(mask, dim=1).type_as(mask) * mask).long() + padding_idx


# ------------------------------------------------------------ grad norms
def multi_tensor_l2_norm(tensors: List[torch.Tensor]) -> torch.Tensor:
    """fp32 L2 norm over a list of tensors; one list-form sum-of-squares launch for all tensors on a
    GPU (the reference uses apex ``multi_tensor_l2norm``: metaseq/utils.py:104-127)."""
    from metaseq_b200.ops import functional as ops

    if not tensors:
        return torch.tensor(0.0)
    dev = tensors[0].device
    if dev.type == "cuda":
        flat = [t.detach().reshape(-1) if t.is_contiguous() else t.detach().contiguous().view(-1) for t in tensors]
        acc = torch.empty(1, dtype=torch.float32, device=dev)
        if len(flat) > 1 and ops.list_kernels_ok(flat):
            ops.sumsq_multi(flat, acc, False)  # the whole list in one launch
        else:
            acc.zero_()
            for t in flat:
                ops.sumsq(t, acc, True)
        return acc.sqrt()[0]
    return torch.norm(torch.stack([torch.norm(t.detach().float()) for t in tensors]))


@torch.no_grad()
def clip_grad_norm_(params, max_norm, norm_type: str = "l2", aggregate_norm_fn=None, device=None) -> torch.Tensor:
    """Clips in place and returns the total norm.  Gradients of FSDP-sharded parameters
    (``p._is_sharded``) are partial: their squared norm is summed over the data-parallel
    group before being combined with the replicated ones; ``aggregate_norm_fn`` then
    folds in the other tensor-parallel ranks."""
    from metaseq_b200.ops import functional as ops
    from metaseq_b200.parallel import utils as dist_utils

    if isinstance(params, torch.Tensor):
        params = [params]
    params = list(params)
    params = [p for p in params if p.grad is not None]
    sharded = [p.grad.detach() for p in params if getattr(p, "_is_sharded", False)]
    local = [p.grad.detach() for p in params if not getattr(p, "_is_sharded", False)]
    if device is None:
        device = params[0].grad.device if params else torch.device("cpu")

    def _norm(grads):
        if not grads:
            return torch.zeros((), dtype=torch.float32, device=device)
        if norm_type == "inf":
            if ops.list_kernels_ok(grads):  # one launch over the list
                return ops.absmax_multi(grads, torch.empty(1, dtype=torch.float32, device=grads[0].device))[0]
            return max(g.abs().max().float() for g in grads)
        return multi_tensor_l2_norm(grads).to(device)

    if norm_type == "inf":
        total = torch.maximum(_norm(sharded), _norm(local)) if (sharded or local) else torch.zeros((), device=device)
        if sharded and dist_utils.is_initialized():
            total = total.clone()
            dist_utils.all_reduce(total, group=dist_utils.get_data_parallel_group(), op="max")
    else:
        sn = _norm(sharded)
        if sharded and dist_utils.is_initialized() and dist_utils.get_data_parallel_world_size() > 1:
            sq = sn.pow(2).clone()
            dist_utils.all_reduce(sq, group=dist_utils.get_data_parallel_group())
            sn = sq.sqrt()
        total = torch.sqrt(sn.pow(2) + _norm(local).pow(2))
    if aggregate_norm_fn is not None:
        total = aggregate_norm_fn(total)
    if max_norm is not None and max_norm > 0:
        coef = (float(max_norm) / (total + 1e-6)).clamp(max=1.0)
        grads = [p.grad.detach() for p in params]
        if ops.list_kernels_ok(grads) and coef.device == grads[0].device:
            # one launch for the whole list, the coefficient read on the device
            ops.scale_multi_(grads, coef.float().reshape(1))
        else:
            for g in grads:
                g.mul_(coef.to(g.dtype) if g.is_floating_point() else coef)
    return total


# ------------------------------------------------------------------ seeds
def set_torch_seed(seed: int):
    assert isinstance(seed, int)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


@contextlib.contextmanager
def numpy_seed(seed, *addl_seeds):
    """Context manager which seeds numpy's global PRNG and restores its state afterwards."""
    if seed is None:
        yield
        return
    if len(addl_seeds) > 0:
        seed = int(hash((seed, *addl_seeds)) % 1e6)
    state = np.random.get_state()
    np.random.seed(seed)
    try:
        yield
    finally:
        np.random.set_state(state)


@contextlib.contextmanager
def torch_seed(seed: int):
    state = torch.get_rng_state()
    cuda_state = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
    set_torch_seed(seed)
    try:
        yield
    finally:
        torch.set_rng_state(state)
        if cuda_state is not None:
            torch.cuda.set_rng_state(cuda_state)


# ------------------------------------------------------------ initialisers
def init_method_normal(sigma: float):
    def init_(tensor):
        return torch.nn.init.normal_(tensor, mean=0.0, std=sigma)

    return init_


def scaled_init_method_normal(sigma: float, num_layers: int):
    """N(0, sigma / sqrt(2 * num_layers)) for the output projections (out_proj, fc2)."""
    std = sigma / math.sqrt(2.0 * num_layers)

    def init_(tensor):
        return torch.nn.init.normal_(tensor, mean=0.0, std=std)

    return init_


# ------------------------------------------------------------ activations
def gelu(x):
    return F.gelu(x.float()).type_as(x)


def relu_squared(x):
    return F.relu(x).pow(2)


def get_activation_fn(name: str) -> Callable:
    if name == "relu":
        return F.relu
    if name == "relu_squared":
        return relu_squared
    if name == "gelu":
        return gelu
    if name == "tanh":
        return torch.tanh
    if name == "linear":
        return lambda x: x
    if name in ("swiglu", "geglu"):
        from metaseq_b200.modules.activation_functions import GatedActivation

        return GatedActivation(name)
    raise RuntimeError(f"--activation-fn {name} not supported")


def get_available_activation_fns() -> List[str]:
    return ["relu", "gelu", "relu_squared", "tanh", "linear", "swiglu", "geglu"]


def softmax(x, dim: int, onnx_trace: bool = False):
    return F.softmax(x, dim=dim, dtype=torch.float32)


def log_softmax(x, dim: int, onnx_trace: bool = False):
    return F.log_softmax(x, dim=dim, dtype=torch.float32)


# ----------------------------------------------------------------- dtypes
def floating_point_precision_convertor(x, fp16: bool, memory_efficient_fp16: bool, bf16: bool):
    if memory_efficient_fp16 or fp16:
        return x.bfloat16() if bf16 else x.half()
    return x.float()


def get_precise_dtype(cfg_common) -> torch.dtype:
    if getattr(cfg_common, "bf16", False):
        return torch.bfloat16
    if getattr(cfg_common, "fp16", False) or getattr(cfg_common, "memory_efficient_fp16", False):
        return torch.float16
    return torch.float32


def has_parameters(module) -> bool:
    try:
        next(module.parameters())
        return True
    except StopIteration:
        return False


# ------------------------------------------------------------ environment
class CudaEnvironment:
    """Snapshot of the current device, gathered across ranks and printed at start-up."""

    def __init__(self):
        cur = torch.cuda.current_device()
        prop = torch.cuda.get_device_properties(f"cuda:{cur}")
        self.name = prop.name
        self.major = prop.major
        self.minor = prop.minor
        self.total_memory_in_GB = prop.total_memory / 1024 / 1024 / 1024

    @staticmethod
    def pretty_print_cuda_env_list(envs):
        num = len(envs)
        center = "CUDA enviroments for all {} workers".format(num)
        banner = 40 - len(center) // 2
        first = "*" * banner + center + "*" * banner
        logger.info(first)
        for r, env in enumerate(envs):
            logger.info(
                "rank {:3d}: capabilities = {:2d}.{:<2d} ; total memory = {:.3f} GB ; name = {:40s}".format(
                    r, env.major, env.minor, env.total_memory_in_GB, env.name
                )
            )
        logger.info(first)


def get_random_port() -> int:
    state = random.getstate()
    random.seed()
    port = random.randint(10_000, 20_000)
    random.setstate(state)
    return port


def tokenize_line(line: str) -> List[str]:
    return re.sub(r"\s+", " ", line).strip().split()


def round_safe(x):
    if torch.is_tensor(x):
        return float(np.round(x.cpu().numpy(), 4))
    try:
        return round(x, 4)
    except Exception:
        return x


def remove_prefix(text: str, prefix: str) -> str:
    return text[len(prefix):] if text.startswith(prefix) else text


def print_r0(*a):
    from metaseq_b200.parallel import utils as dist_utils

    if dist_utils.get_global_rank() == 0:
        print(*a, flush=True)


def get_env(name, default=None):
    return os.environ.get(name, default)


# ------------------------------------------------ further helpers of the reference's utils module
def split_paths(paths: str) -> List[str]:
    """``a:b`` (``os.pathsep``) for local paths, ``a|b`` when the entries are URLs (metaseq/utils.py:36)."""
    return paths.split("|") if "://" in paths else paths.split(os.pathsep)


def fill_with_neg_inf(t: torch.Tensor) -> torch.Tensor:
    """``t`` filled with -inf in place, for any floating dtype (metaseq/utils.py:232)."""
    return t.fill_(float("-inf"))


def get_perplexity(loss, round: int = 2, base: float = 2):
    """``base ** loss`` rounded; 0 for a missing loss, inf when the power overflows (metaseq/utils.py:340)."""
    if loss is None:
        return 0.0
    try:
        value = base ** float(loss)
    except OverflowError:
        return float("inf")
    return builtins.round(value, round) if math.isfinite(value) else value


def get_precise_epoch(epoch: Optional[int], count: int, iterator_size: int) -> Optional[float]:
    """Fractional epoch after ``count + 1`` of ``iterator_size`` batches (metaseq/utils.py:494)."""
    if epoch is None or iterator_size <= 0:
        return None
    return epoch - 1 + (count + 1) / float(iterator_size)


def get_model_init_dtype(args) -> torch.dtype:
    """Parameters are created in 16 bits when nothing keeps an fp32 copy of them (metaseq/utils.py:486)."""
    if getattr(args, "memory_efficient_fp16", False) or getattr(args, "inference", False):
        return torch.bfloat16 if getattr(args, "bf16", False) else torch.float16
    return torch.float32


def get_rng_state() -> Dict[str, torch.Tensor]:
    state = {"torch_rng_state": torch.get_rng_state()}
    if torch.cuda.is_available():
        state["cuda_rng_state"] = torch.cuda.get_rng_state()
    return state


def set_rng_state(state: Dict[str, torch.Tensor]) -> None:
    torch.set_rng_state(state["torch_rng_state"])
    if torch.cuda.is_available() and "cuda_rng_state" in state:
        torch.cuda.set_rng_state(state["cuda_rng_state"])


@contextlib.contextmanager
def set_rank_seed(seed: int, update: int):
    """Seeds torch, numpy and ``random`` with ``seed + update * world + rank`` inside the block and restores all
    three generators afterwards: every rank and every update draws its own stream (metaseq/utils.py:388-410)."""
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        rank, world = torch.distributed.get_rank(), torch.distributed.get_world_size()
    else:
        rank, world = 0, 1
    rank_seed = seed + update * world + rank
    torch_state, np_state, py_state = get_rng_state(), np.random.get_state(), random.getstate()
    torch.manual_seed(rank_seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(rank_seed)
    np.random.seed(rank_seed % (2 ** 32))
    random.seed(rank_seed)
    try:
        yield rank_seed
    finally:
        random.setstate(py_state)
        np.random.set_state(np_state)
        set_rng_state(torch_state)


def multi_tensor_l2_total_norm(grads, chunk_size: int = 2048 * 32) -> torch.Tensor:
    """Norm over tensors that may live on several devices: one fused norm per device, combined on the first
    (metaseq/utils.py:104-131).  ``chunk_size`` is accepted for call compatibility."""
    by_device: Dict[torch.device, List[torch.Tensor]] = {}
    for g in grads:
        by_device.setdefault(g.device, []).append(g)
    if not by_device:
        return torch.tensor(0.0)
    first = next(iter(by_device))
    norms = [multi_tensor_l2_norm(ts).to(first) for ts in by_device.values()]
    return torch.norm(torch.stack(norms))


def resolve_max_positions(*limits):
    """Element-wise smallest of several position limits.  A limit is a number, a tuple of numbers (one per stream)
    or a dict of them; ``None`` (a whole limit or an entry) means "no constraint"; a number meets a tuple or a dict
    by applying to every entry (metaseq/utils.py:259-293)."""

    def smallest(a, b):
        if a is None:
            return b
        if b is None:
            return a
        return min(a, b)

    def broadcast(number, shape):
        if isinstance(shape, tuple):
            return tuple(number for _ in shape)
        if isinstance(shape, dict):
            return {k: broadcast(number, v) for k, v in shape.items()}
        return number

    def merge(a, b):
        if isinstance(a, (int, float)) and not isinstance(b, (int, float)):
            a = broadcast(a, b)
        elif isinstance(b, (int, float)) and not isinstance(a, (int, float)):
            b = broadcast(b, a)
        if isinstance(a, dict):
            out = copy.deepcopy(a)
            for k, v in b.items():
                out[k] = merge(out[k], v) if k in out and out[k] is not None and v is not None else smallest(out.get(k), v)
            return out
        if isinstance(a, (tuple, list)):
            return tuple(smallest(x, y) for x, y in zip(a, b))
        return smallest(a, b)

    result = None
    for limit in limits:
        if limit is None:
            continue
        result = limit if result is None else merge(result, limit)
    return result


def import_user_module(args) -> None:
    """Imports the package named by ``args.user_dir`` once, so that the components it registers exist before the
    command line is parsed.  A relative path is also tried against this package and its parent; a module name that
    is already imported from elsewhere is an error (metaseq/utils.py:296-329)."""
    path = getattr(args, "user_dir", None)
    if path is None:
        return
    candidates = [os.path.abspath(path)]
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    candidates += [os.path.join(here, path), os.path.join(os.path.dirname(here), path)]
    found = next((c for c in candidates if os.path.exists(c)), None)
    if found is None:
        raise FileNotFoundError(candidates[0])
    memo = import_user_module.__dict__.setdefault("memo", set())
    if found in memo:
        return
    memo.add(found)
    parent, name = os.path.split(found.rstrip(os.sep))
    if name in sys.modules:
        raise ImportError(f"Failed to import --user-dir={found}: a module called {name!r} is already imported; "
                          "rename the directory to something unique")
    sys.path.insert(0, parent)
    importlib.import_module(name)


def get_token_to_word_mapping(tokens, exclude_list) -> Dict[int, int]:
    """Position -> running count of tokens that are not in ``exclude_list`` (metaseq/utils.py:541)."""
    counts = itertools.accumulate(int(t not in exclude_list) for t in tokens)
    return dict(enumerate(counts))


def extract_hard_alignment(attn: torch.Tensor, src_sent, tgt_sent, pad: int, eos: int):
    """For every real target token the source word with the largest attention weight, as (source word, target
    word) pairs counted from 0.  ``attn``: [target, source] (metaseq/utils.py:549-570)."""
    tgt_valid = ((tgt_sent != pad) & (tgt_sent != eos)).nonzero(as_tuple=False).squeeze(-1)
    src_invalid = ((src_sent == pad) | (src_sent == eos)).nonzero(as_tuple=False).squeeze(-1)
    if len(tgt_valid) == 0 or len(src_invalid) >= len(src_sent):
        return []
    src_word = get_token_to_word_mapping(src_sent, [eos, pad])
    tgt_word = get_token_to_word_mapping(tgt_sent, [eos, pad])
    weights = attn[tgt_valid].clone()
    weights[:, src_invalid] = float("-inf")
    best = weights.argmax(dim=1)
    return [(src_word[int(s)] - 1, tgt_word[int(t)] - 1) for t, s in zip(tgt_valid.tolist(), best.tolist())]


def extract_soft_alignment(attn: torch.Tensor, src_sent, tgt_sent, pad: int, eos: int):
    """Attention rows of the non-pad target tokens over the non-pad source tokens, formatted with six decimals
    (metaseq/utils.py:573-582)."""
    tgt_valid = (tgt_sent != pad).nonzero(as_tuple=False)
    src_valid = (src_sent != pad).nonzero(as_tuple=False).squeeze(-1)
    if len(tgt_valid) == 0 or len(src_valid) == 0:
        return []
    return [[f"{p:.6f}" for p in row.tolist()] for row in attn[tgt_valid, src_valid]]
