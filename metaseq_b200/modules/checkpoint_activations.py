"""Activation checkpointing for arbitrary modules: ``checkpoint_wrapper(m)`` makes ``m.forward``
keep only its inputs and recompute the rest during backward, restoring the default and the
tensor-parallel RNG streams so dropout repeats exactly; saved inputs can optionally be moved
to the host (``offload_to_cpu``) or kept as a 1/tp slice per tensor-parallel rank and gathered
back in backward (``distribute_checkpointed_activations``).  Reference:
metaseq/modules/checkpoint_activation_wrapper/checkpoint_activations.py:104-411.

The decoder layer's fused path has recomputation built in (``LayerSpec.recompute``); this
wrapper serves the modular path and user modules."""
from __future__ import annotations

import contextlib
import functools
import threading
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from metaseq_b200.parallel import mpu


class _State(threading.local):
    def __init__(self):
        self.disabled = False      # wrappers run their module directly
        self.checkpointing = False  # inside the no-grad first pass of a wrapped module
        self.recomputing = False    # inside the recomputation during backward


_state = _State()


@contextlib.contextmanager
def _flag(name: str, value: bool = True):
    before = getattr(_state, name)
    setattr(_state, name, value)
    try:
        yield
    finally:
        setattr(_state, name, before)


def disable_checkpointing():
    """Context in which wrapped modules keep their activations (e.g. a forward pass for evaluation or for a
    consumer that needs no backward); reference :41-48."""
    return _flag("disabled")


def enable_checkpointing():
    return _flag("checkpointing")


def enable_recomputing():
    return _flag("recomputing")


def is_checkpointing_disabled() -> bool:
    return _state.disabled


def is_checkpointing() -> bool:
    """True during the first (activation-dropping) pass of a wrapped module."""
    return _state.checkpointing


def is_recomputing() -> bool:
    """True while backward re-runs a wrapped module: modules with side effects in ``forward`` (counters, running
    statistics) check it to apply them once."""
    return _state.recomputing


def checkpoint_wrapper(module: nn.Module, offload_to_cpu: bool = False,
                       distribute_checkpointed_activations: bool = False) -> nn.Module:
    module._checkpoint_orig_forward = module.forward
    module.forward = functools.partial(_checkpointed_forward, module, offload_to_cpu,
                                       distribute_checkpointed_activations)
    return module


def checkpoint(fn, owner: nn.Module, *args, offload_to_cpu: bool = False,
               distribute_checkpointed_activations: bool = False, **kwargs):
    """Functional form: ``fn(*args, **kwargs)`` with only its tensor arguments kept for backward, where ``fn`` is
    run again.  ``owner`` is the module whose parameters ``fn`` reads (it decides whether anything needs a gradient)."""
    shim = _Shim()
    shim._checkpoint_orig_forward, shim.parameters = fn, owner.parameters
    return _checkpointed_forward(shim, offload_to_cpu, distribute_checkpointed_activations, *args, **kwargs)


class _Shim:
    pass


def _checkpointed_forward(module, offload_to_cpu, distribute, *args, **kwargs):
    flat_kwargs_keys = list(kwargs.keys())
    flat = list(args) + [kwargs[k] for k in flat_kwargs_keys]
    tensors = [(i, a) for i, a in enumerate(flat) if torch.is_tensor(a)]
    others = {i: a for i, a in enumerate(flat) if not torch.is_tensor(a)}
    meta = {"n_args": len(args), "kw_keys": flat_kwargs_keys, "others": others,
            "tensor_idx": [i for i, _ in tensors], "offload": offload_to_cpu, "distribute": distribute}
    if _state.disabled or not torch.is_grad_enabled() or not any(t.requires_grad for _, t in tensors) and \
            not any(p.requires_grad for p in module.parameters()):
        return module._checkpoint_orig_forward(*args, **kwargs)
    dummy = torch.zeros(1, requires_grad=True) if not any(t.requires_grad for _, t in tensors) else None
    out = _CheckpointFn.apply(module._checkpoint_orig_forward, meta, dummy, *[t for _, t in tensors])
    return out


def _rng_state():
    st = {"cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    st["tracker"] = mpu.get_cuda_rng_tracker().get_states()
    return st


def _set_rng_state(st):
    torch.set_rng_state(st["cpu"])
    if "cuda" in st:
        torch.cuda.set_rng_state(st["cuda"])
    mpu.get_cuda_rng_tracker().set_states(st["tracker"])


def is_autocast_enabled() -> bool:
    """Whether the GPU autocast mode is on (the recomputation must run under the mode of the first pass)."""
    return torch.is_autocast_enabled()


@contextlib.contextmanager
def autocast(enabled: bool):
    """Re-enters (or leaves) GPU autocast for the recomputation; a no-op where it is already in that state."""
    if enabled and torch.cuda.is_available():
        with torch.autocast("cuda", enabled=True):
            yield
    elif not enabled and torch.is_autocast_enabled():
        with torch.autocast("cuda", enabled=False):
            yield
    else:
        yield


def _rebuild(meta, tensors):
    flat = [None] * (len(meta["tensor_idx"]) + len(meta["others"]))
    for i, t in zip(meta["tensor_idx"], tensors):
        flat[i] = t
    for i, o in meta["others"].items():
        flat[i] = o
    args = flat[: meta["n_args"]]
    kwargs = dict(zip(meta["kw_keys"], flat[meta["n_args"]:]))
    return args, kwargs


class _CheckpointFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_fn, meta, dummy, *tensors):
        ctx.run_fn = run_fn
        ctx.meta = meta
        ctx.rng = _rng_state()
        ctx.had_autocast = is_autocast_enabled()
        ctx.devices = [t.device for t in tensors]
        ctx.grad_flags = [t.requires_grad for t in tensors]
        saved = []
        ctx.shapes = [None] * len(tensors)
        for i, t in enumerate(tensors):
            s = t.detach()
            if meta["distribute"] and i == 0 and mpu.get_tensor_model_parallel_world_size() > 1 and \
                    s.numel() % mpu.get_tensor_model_parallel_world_size() == 0:
                ctx.shapes[i] = s.shape
                s = mpu.split_tensor_into_1d_equal_chunks(s.contiguous()).clone()
            if meta["offload"]:
                s = s.to("cpu", non_blocking=True)
            saved.append(s)
        ctx.save_for_backward(*saved)
        with torch.no_grad(), enable_checkpointing():
            args, kwargs = _rebuild(meta, tensors)
            out = run_fn(*args, **kwargs)
        ctx.out_is_tuple = isinstance(out, tuple)
        return out

    @staticmethod
    def backward(ctx, *grads):
        saved = list(ctx.saved_tensors)
        inputs = []
        for i, s in enumerate(saved):
            if ctx.meta["offload"]:
                s = s.to(ctx.devices[i], non_blocking=True)
            if ctx.shapes[i] is not None:
                s = mpu.gather_split_1d_tensor(s).view(ctx.shapes[i])
            s = s.detach().requires_grad_(ctx.grad_flags[i])
            inputs.append(s)
        now = _rng_state()
        _set_rng_state(ctx.rng)
        with torch.enable_grad(), enable_recomputing(), autocast(ctx.had_autocast):
            args, kwargs = _rebuild(ctx.meta, inputs)
            out = ctx.run_fn(*args, **kwargs)
        _set_rng_state(now)
        outs = out if isinstance(out, tuple) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        in_grads = tuple(t.grad if t.requires_grad else None for t in inputs)
        return (None, None, None) + in_grads


# the reference's public names for the pieces above (metaseq/modules/checkpoint_activation_wrapper/
# checkpoint_activations.py:30, :235-262, :265)
ThreadLocal = _State
CheckpointFunction = _CheckpointFn
get_rng_state = _rng_state
set_rng_state = _set_rng_state
