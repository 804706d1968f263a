"""Fully sharded data parallelism (ZeRO-3 / ZeRO-2 style) written against plain
``torch.distributed``.

What the reference gets from fairscale's ``FullyShardedDataParallel`` through
metaseq/distributed/fully_sharded_data_parallel.py:28-152 is provided here natively:

* every wrapped unit flattens its own parameters (those not owned by a nested unit) into one
  flat tensor, pads it to a multiple of the data-parallel world size and keeps only this
  rank's equal-sized shard as the trainable ``flat_param`` (``flat_param_0`` in state dicts);
* before a unit's forward the shards are all-gathered into a full flat buffer and the
  module's parameters become views into it; with ``reshard_after_forward`` the buffer is
  dropped after forward and gathered again for backward, otherwise it is kept until the
  optimizer step (``--no-reshard-after-forward``, what the OPT runs use);
* gradients are written straight into a full flat gradient buffer (``_grad_view`` of each
  parameter view, see ``metaseq_b200.ops.autograd._direct_grad``) and reduce-scattered to the
  owning ranks when the unit's backward finishes;
* ``local_state_dict`` / ``shard_metadata`` reproduce the on-disk layout the checkpoint tools
  expect (names / shapes / numels / padding per flat parameter, padding at the end).

Communication runs on a side stream: the all-gathers of all units are queued at the start of
the step in forward order and each unit waits only for its own, reduce-scatters are queued as
units finish backward; compute never waits for a collective it does not need.  The NCCL calls
can be replaced by the fused peer-memory kernels through ``comm`` (``metaseq_b200.parallel.symm``).
"""
from __future__ import annotations

import contextlib
import functools
import logging
import os
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

logger = logging.getLogger(__name__)


class DummyProcessGroup:
    """Stand-in group of size 1 (offline tools that instantiate sharded models on one process)."""

    def __init__(self, rank: int = 0, size: int = 1):
        self._rank, self._size = rank, size

    def rank(self):
        return self._rank

    def size(self):
        return self._size


def _group_size(group) -> int:
    if group is None:
        return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    if isinstance(group, DummyProcessGroup):
        return group.size()
    return dist.get_world_size(group=group)


def _group_rank(group) -> int:
    if group is None:
        return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    if isinstance(group, DummyProcessGroup):
        return group.rank()
    return dist.get_rank(group=group)


class _UnitInput(torch.autograd.Function):
    """Identity on the unit's input.  Its backward runs when the gradient w.r.t. the input is
    ready, i.e. after every parameter gradient of the unit has been produced."""

    @staticmethod
    def forward(ctx, unit, x):
        ctx.unit = unit
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.unit._post_backward()
        return None, g


class _UnitOutput(torch.autograd.Function):
    """Identity on the unit's output.  Its backward runs before the unit's own backward: the
    place to re-gather parameters and to arm the end-of-backward callback."""

    @staticmethod
    def forward(ctx, unit, y):
        ctx.unit = unit
        return y.view_as(y)

    @staticmethod
    def backward(ctx, g):
        ctx.unit._pre_backward()
        return None, g


class FullyShardedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, process_group=None, reshard_after_forward: bool = True,
                 mixed_precision: bool = False, fp32_reduce_scatter: bool = False, flatten_parameters: bool = True,
                 cpu_offload: bool = False, compute_dtype: Optional[torch.dtype] = None, bucket_cap_mb: int = 25,
                 state_dict_device=None, gradient_predivide_factor: Optional[float] = None,
                 use_sharded_state: bool = False, comm=None, **unused):
        super().__init__()
        self.process_group = process_group
        self.world_size = _group_size(process_group)
        self.rank = _group_rank(process_group)
        self.reshard_after_forward = reshard_after_forward and self.world_size > 1
        self.mixed_precision = mixed_precision
        self.fp32_reduce_scatter = fp32_reduce_scatter
        self.compute_dtype = compute_dtype
        self.use_sharded_state = use_sharded_state
        self.state_dict_device = state_dict_device
        # ``cpu_offload``: the trainable shard, its gradient and the optimizer state live in (pinned) host memory;
        # the shard is copied to the compute device for every gather and the reduced gradient copied back
        self.cpu_offload = bool(cpu_offload)
        # ``comm``: a ``PeerComm``, or "fused" (one is built for the process group at first use, CUDA and
        # world size > 1 only), or None / "nccl" for torch.distributed collectives
        self.comm = comm if not isinstance(comm, str) else None
        self._comm_request = comm if isinstance(comm, str) else None
        if gradient_predivide_factor is None:
            gradient_predivide_factor = self._default_predivide(self.world_size)
        self.gradient_predivide_factor = float(gradient_predivide_factor)
        self.gradient_postdivide_factor = self.world_size / self.gradient_predivide_factor
        self.module = module
        self._is_root: Optional[bool] = None
        self._full_param: Optional[torch.Tensor] = None
        self._full_grad: Optional[torch.Tensor] = None
        self._views: List[torch.Tensor] = []
        self._gather_event = None
        self._reduce_pending = False
        self._backward_armed = False
        self._post_backward_done = True
        self._needs_gather = True
        self._flatten_own_params()

    @staticmethod
    def _default_predivide(world_size: int) -> float:
        factor = 1
        while world_size % factor == 0 and world_size / factor > factor:
            factor *= 2
        return float(factor)

    # ------------------------------------------------------------ flattening
    def _own_named_params(self):
        """(owner module, attribute name, full dotted name, param) for parameters not owned by a
        nested FSDP unit, shared parameters listed once (first occurrence)."""
        nested = set()
        for m in self.module.modules():
            if isinstance(m, FullyShardedDataParallel):
                for sub in m.modules():
                    nested.add(id(sub))
        seen = {}
        out, shared = [], []
        for mod_name, mod in self.module.named_modules():
            if id(mod) in nested:
                continue
            for pname, p in list(mod._parameters.items()):
                if p is None:
                    continue
                full = _clean_name(f"{mod_name}.{pname}" if mod_name else pname)
                if id(p) in seen:
                    shared.append((full, seen[id(p)][0], mod, pname, seen[id(p)][1]))
                    continue
                seen[id(p)] = (full, len(out))
                out.append((mod, pname, full, p))
        return out, shared

    def _flatten_own_params(self):
        own, shared = self._own_named_params()
        self._param_infos = [(mod, pname) for mod, pname, _, _ in own]
        self._shared_infos = [(mod, pname, idx) for (_, _, mod, pname, idx) in shared]
        self.param_names = [full for _, _, full, _ in own]
        self.param_shapes = [p.shape for _, _, _, p in own]
        self.param_numels = [p.numel() for _, _, _, p in own]
        self.shared_param_info = [(a, b) for (a, b, _, _, _) in shared]
        self.has_params = len(own) > 0
        if not self.has_params:
            self.flat_param = None
            self.padding = 0
            return
        dtype = own[0][3].dtype
        device = own[0][3].device
        total = sum(self.param_numels)
        self.unpadded_numel = total
        shard = (total + self.world_size - 1) // self.world_size
        # keep every view 16-byte aligned inside the gathered buffer and shards a multiple of 8 elements
        shard = (shard + 7) // 8 * 8
        self.shard_numel = shard
        self.padded_numel = shard * self.world_size
        self.padding = self.padded_numel - total  # lives at the end of the last shard(s)
        flat = torch.zeros(self.padded_numel, dtype=dtype, device=device)
        off = 0
        for _, _, _, p in own:
            flat[off:off + p.numel()].copy_(p.data.reshape(-1))
            off += p.numel()
        local = flat[self.rank * shard:(self.rank + 1) * shard].clone()
        if self.cpu_offload:
            # compute where the module was built, or on the current GPU when it was built on the host
            self._offload_compute_device = device if device.type != "cpu" or not torch.cuda.is_available() \
                else torch.device("cuda", torch.cuda.current_device())
            local = local.cpu()
            if torch.cuda.is_available():
                local = local.pin_memory()
        self.flat_param = nn.Parameter(local)
        self.flat_param._is_sharded = self.world_size > 1
        self.flat_param._fsdp_unit = self
        any_mp = any(getattr(p, "model_parallel", False) for _, _, _, p in own)
        self.flat_param.model_parallel = any_mp
        for mod, pname, _, p in own:
            del mod._parameters[pname]
        for mod, pname, _ in self._shared_infos:
            if pname in mod._parameters:
                del mod._parameters[pname]
        del flat
        self._set_views(None)

    # ------------------------------------------------------------------ views
    def _set_views(self, full: Optional[torch.Tensor]):
        """Points the module's parameter attributes at views of ``full`` (or at empty
        placeholders when ``None``).  Views are created once per full buffer and stay valid
        while its storage is released and re-filled, so tensors saved by autograd see the
        re-gathered values."""
        self._views = []
        off = 0
        for (mod, pname), shape, n in zip(self._param_infos, self.param_shapes, self.param_numels):
            if full is None:
                v = torch.empty(0, dtype=self.flat_param.dtype, device=self._compute_device)
            else:
                v = full[off:off + n].view(shape)
                v.requires_grad_(self.flat_param.requires_grad)
            mod.__dict__[pname] = v
            self._views.append(v)
            off += n
        for mod, pname, idx in self._shared_infos:
            mod.__dict__[pname] = self._views[idx]
        self._ready_handle = None
        if full is not None and self.comm is not None and self.world_size > 1:
            # matrices carry the arrival flags of their chunks: the GEMMs that read them wait per tile inside
            # the kernel, and only the chunks holding the small (non-matrix) parameters are awaited up front
            inner = self.module
            while not getattr(inner, "supports_operand_flags", False) and hasattr(inner, "module"):
                inner = inner.module  # activation-checkpoint and similar wrappers
            flagged = set(getattr(inner, "operand_flag_parameters", ())) \
                if getattr(inner, "supports_operand_flags", False) else set()
            if flagged:
                handle = self.comm.ready_handle(full)
                handle.active = False
                esz = full.element_size()
                off, small = 0, []
                for v, n, name in zip(self._views, self.param_numels, self.param_names):
                    if any(name == f or name.endswith("." + f) for f in flagged) and v.dim() == 2:
                        v._msq_ready = handle
                    else:
                        small.append((off * esz, (off + n) * esz))
                    off += n
                self._ready_handle = handle
                self._small_param_ranges = tuple(small)
        self._refresh_grad_views()

    def _refresh_grad_views(self):
        off = 0
        for v, n, shape in zip(self._views, self.param_numels, self.param_shapes):
            if self._full_grad is not None and v.numel() == n:
                v._grad_view = self._full_grad[off:off + n].view(shape)
                if not hasattr(v, "_grad_filled"):
                    v._grad_filled = False
            elif hasattr(v, "_grad_view"):
                del v._grad_view
            off += n

    def _compute_dtype(self):
        if self.mixed_precision and self.compute_dtype is not None:
            return self.compute_dtype
        return self.flat_param.dtype

    # ----------------------------------------------------------------- gather
    def _comm_stream(self):
        root = self._root()
        if getattr(root, "_side_stream", None) is None and self.flat_param is not None \
                and self._compute_device.type == "cuda":
            root._side_stream = torch.cuda.Stream()
        return getattr(root, "_side_stream", None)

    def _root(self) -> "FullyShardedDataParallel":
        return self.__dict__.get("_root_ref") or self

    @property
    def _compute_device(self) -> torch.device:
        """Where gathered parameters and gradients live: the shard's own device unless the shard is offloaded."""
        if self.cpu_offload:
            return self._offload_compute_device
        return self.flat_param.device

    def _aliases_shard(self) -> bool:
        return self.world_size == 1 and self._compute_dtype() == self.flat_param.dtype \
            and self.flat_param.device == self._compute_device

    def _gather_full(self, asynchronous: bool = False):
        """Makes the full flat parameter current (idempotent until ``_needs_gather`` is set)."""
        if not self.has_params:
            return
        cdt = self._compute_dtype()
        src = self.flat_param.data
        if src.device != self._compute_device:
            src = src.to(self._compute_device, non_blocking=True)  # offloaded shard: host -> device per gather
        if self._aliases_shard():
            if self._full_param is None or self._full_param.data_ptr() != src.data_ptr():
                self._full_param = src
                self._set_views(src)
            self._needs_gather = False
        else:
            nbytes = self.padded_numel * torch.empty((), dtype=cdt).element_size()
            if self._full_param is None:
                if self.comm is not None:
                    # symmetric memory: peers store their shards straight into this buffer; it stays
                    # allocated (the gathered copy is re-filled in place after every optimizer step)
                    self._full_param = self.comm.alloc_full(self.padded_numel, cdt)
                else:
                    self._full_param = torch.empty(self.padded_numel, dtype=cdt, device=src.device)
                self._set_views(self._full_param)
                self._needs_gather = True
            elif self._full_param.untyped_storage().size() == 0:
                self._full_param.untyped_storage().resize_(nbytes)
                self._needs_gather = True
            if self._needs_gather:
                # ``.data`` aliases the storage under a separate version counter: re-filling the buffer between
                # forward and backward must not invalidate the views autograd saved
                full = self._full_param.data
                local = src if src.dtype == cdt else src.to(cdt)
                if self.world_size == 1:
                    full[: local.numel()].copy_(local)
                else:
                    stream = self._comm_stream() if (asynchronous and src.is_cuda) else None
                    if self.comm is not None:
                        self.comm.all_gather(full, local, stream=stream, wait=False)
                        self._gather_flags_pending = True
                    elif stream is not None:
                        stream.wait_stream(torch.cuda.current_stream())
                        with torch.cuda.stream(stream):
                            dist.all_gather_into_tensor(full, local, group=self.process_group)
                            ev = torch.cuda.Event()
                            ev.record(stream)
                        self._gather_event = ev
                        local.record_stream(stream)
                    else:
                        dist.all_gather_into_tensor(full, local, group=self.process_group)
                self._needs_gather = False
        if self._full_grad is None and self.flat_param.requires_grad and torch.is_grad_enabled():
            self._alloc_full_grad()

    def _alloc_full_grad(self):
        """The unit's flat gradient buffer: a slice of one arena shared by all units of the root, allocated
        (zeroed) once.  It is never cleared again: the first gradient written to a view in a step overwrites,
        and views that received nothing are zeroed individually before the reduction."""
        cdt = self._compute_dtype()
        root = self._root()
        arena = root.__dict__.get("_grad_arena")
        if arena is None or arena.dtype != cdt or arena.device != self._compute_device:
            units = [u for u in (root.__dict__.get("_units") or [self]) if u.has_params and u.flat_param.requires_grad]
            if self not in units:
                units.append(self)
            total, offs = 0, {}
            for u in units:
                offs[id(u)] = total
                total += (u.padded_numel + 127) // 128 * 128
            comm = root.__dict__.get("_peer_comm")
            if comm is not None and comm.pulls_gradients and all(u.comm is comm for u in units):
                # owners read every rank's gradients in place over NVLink: same offset in every rank's region
                arena = comm.alloc_symmetric(total, cdt)
            else:
                arena = torch.zeros(total, dtype=cdt, device=self._compute_device)
            root.__dict__["_grad_arena"] = arena
            root.__dict__["_grad_arena_offsets"] = offs
        off = root.__dict__["_grad_arena_offsets"].get(id(self))
        if off is None:
            self._full_grad = torch.zeros(self.padded_numel, dtype=cdt, device=self._compute_device)
        else:
            self._full_grad = arena[off:off + self.padded_numel]
        for v in self._views:
            v._grad_filled = False
        self._refresh_grad_views()

    def _wait_gather(self):
        if getattr(self, "_gather_flags_pending", False):
            handle = self.__dict__.get("_ready_handle")
            if handle is not None and os.environ.get("MSQ_FSDP_GEMM_WAIT", "1") == "1":
                # small parameters now; each weight matrix when (and where) its GEMM loads it
                handle.active = self.comm.wait_byte_ranges(self._full_param, self._small_param_ranges)
            else:
                self.comm.wait_gathered(self._full_param)  # one kernel polling every chunk's flag
            self._gather_flags_pending = False
        if self._gather_event is not None:
            torch.cuda.current_stream().wait_event(self._gather_event)
            self._gather_event = None

    def _free_full(self):
        """Releases the storage of the gathered copy (the tensor object and its views survive)."""
        if self._full_param is None or self._aliases_shard() or self.comm is not None:
            return
        self._wait_gather()
        self._full_param.untyped_storage().resize_(0)
        self._needs_gather = True

    # ---------------------------------------------------------------- forward
    def _lazy_init(self):
        if self._is_root is not None:
            return
        self._is_root = True
        self._side_stream = None
        self._units = [m for m in self.modules() if isinstance(m, FullyShardedDataParallel)]
        for u in self._units:
            if u is not self:
                u._is_root = False
                object.__setattr__(u, "_root_ref", self)  # plain attribute: not a submodule
        self._step_gathered = False
        self._build_comm()

    def _build_comm(self):
        """One ``PeerComm`` for all units when the fused communication backend was requested."""
        units = [u for u in self._units if u.has_params and u._comm_request == "fused" and u.comm is None
                 and u.world_size > 1 and u._compute_device.type == "cuda"]
        if units and self.reshard_after_forward:
            # the peer-memory collectives fill gathered copies that stay resident in symmetric memory; a model
            # that asks for its gathered parameters to be dropped after forward gets the library collectives
            logger.warning("--comm-backend fused keeps gathered parameters resident (use --no-reshard-after-forward); "
                           "reshard-after-forward was requested, so FSDP uses NCCL collectives")
            return
        if not units:
            return
        from .symm import PeerComm

        need = 0
        for u in units:
            esz = torch.empty((), dtype=u._compute_dtype()).element_size()
            # gathered copy + either the reduce-scatter landing slots or (pull transport) the unit's part of the
            # gradient arena, which then lives in symmetric memory
            need += 2 * (u.padded_numel * esz + 2048)
        comm = PeerComm(units[0].process_group, units[0]._compute_device, heap_bytes=need + (1 << 20))
        for u in units:
            u.comm = comm
        self._peer_comm = comm

    def prefetch_all(self):
        """Queues the all-gathers of every unit, in module order, on the communication stream."""
        self._lazy_init()
        comm = self.__dict__.get("_peer_comm")
        if comm is not None:
            # one stream hand-over for all units, then one native call per unit
            items = []
            for u in self._units:
                if not u.has_params:
                    continue
                first = u._full_param is None
                if first:
                    u._full_param = comm.alloc_full(u.padded_numel, u._compute_dtype())
                    u._set_views(u._full_param)
                    u._needs_gather = True
                if u._needs_gather:
                    src = u.flat_param.data
                    if src.device != u._compute_device:
                        src = src.to(u._compute_device, non_blocking=True)
                    cdt = u._compute_dtype()
                    items.append((u._full_param, src if src.dtype == cdt else src.to(cdt)))
                    u._needs_gather = False
                    u._gather_flags_pending = True
                if u._full_grad is None and u.flat_param.requires_grad and torch.is_grad_enabled():
                    u._alloc_full_grad()
            if items:
                comm.all_gather_many(items, self._comm_stream())
            return
        for u in self._units:
            u._gather_full(asynchronous=True)

    @property
    def unwrapped_module(self) -> nn.Module:
        """The module that was wrapped (this engine keeps it as is; parameters are views of the flat buffers)."""
        return self.module

    def forward(self, *args, **kwargs):
        self._lazy_init()
        if self._is_root and self.world_size > 1 and not self._step_gathered and not self.reshard_after_forward:
            self.prefetch_all()
            self._step_gathered = True
        self._gather_full()
        self._wait_gather()
        grad_mode = torch.is_grad_enabled() and self.has_params and self.flat_param.requires_grad
        if grad_mode:
            self._post_backward_done = False
            args = tuple(_UnitInput.apply(self, a) if (torch.is_tensor(a) and a.requires_grad) else a for a in args)
            self._input_hooked = any(torch.is_tensor(a) and a.requires_grad for a in args)
        out = self.module(*args, **kwargs)
        if grad_mode:
            out = _map_first_tensor(out, lambda t: _UnitOutput.apply(self, t))
        if self.reshard_after_forward:
            self._free_full()
        handle = self.__dict__.get("_ready_handle")
        if handle is not None and handle.active:
            # every matrix of the unit has been consumed at least once: later readers (backward) need no polling
            handle.active = False
        return out

    # --------------------------------------------------------------- backward
    def _pre_backward(self):
        root = self._root()
        if not root._backward_armed:
            root._backward_armed = True
            torch.autograd.Variable._execution_engine.queue_callback(root._finish_backward)
        if self.reshard_after_forward:
            self._gather_full()
            self._wait_gather()

    def _post_backward(self):
        """All gradients of this unit are in ``_full_grad`` (or on the views): reduce them."""
        if self._post_backward_done or not self.has_params:
            return
        self._post_backward_done = True
        self._collect_view_grads()
        if self._full_grad is None:
            return
        for v in self._views:
            if not getattr(v, "_grad_filled", True) and hasattr(v, "_grad_view"):
                v._grad_view.zero_()  # parameter without a gradient this step: the buffer still holds the last one
                v._grad_filled = True
        full_grad = self._full_grad
        if self.world_size == 1:
            same = full_grad.dtype == self.flat_param.dtype
            shard = full_grad if same else full_grad.to(self.flat_param.dtype)
            # the flat buffer doubles as the parameter's gradient only when no cast (or host copy) sits in between;
            # otherwise each micro-batch's buffer is added to the parameter's gradient and then overwritten
            self._accumulate_shard_grad(shard, owns_buffer=same)
            if self.flat_param.grad is None or self.flat_param.grad.data_ptr() != full_grad.data_ptr():
                for v in self._views:
                    if hasattr(v, "_grad_filled"):
                        v._grad_filled = False
        elif self.comm is not None:
            # peer-memory reduce-scatter: slices are pushed to their owners and summed there in fp32 with the
            # 1 / world_size factor applied once, so neither pre-division nor an fp32 copy is needed
            shard = torch.empty(self.shard_numel, dtype=self.flat_param.dtype, device=full_grad.device)
            self.comm.reduce_scatter(shard, full_grad, key=self._full_param, stream=self._comm_stream(),
                                     scale=1.0 / self.world_size)
            self._root()._reduce_pending = True
            self._accumulate_shard_grad(shard, owns_buffer=False)
        else:
            if self.fp32_reduce_scatter and full_grad.dtype != torch.float32:
                full_grad = full_grad.float()
            if self.gradient_predivide_factor > 1:
                full_grad.div_(self.gradient_predivide_factor)
            shard = torch.empty(self.shard_numel, dtype=full_grad.dtype, device=full_grad.device)
            stream = self._comm_stream() if full_grad.is_cuda else None
            if stream is not None:
                stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(stream):
                    dist.reduce_scatter_tensor(shard, full_grad, group=self.process_group)
                    if self.gradient_postdivide_factor > 1:
                        shard.div_(self.gradient_postdivide_factor)
                full_grad.record_stream(stream)
                shard.record_stream(stream)
                self._root()._reduce_pending = True
            else:
                dist.reduce_scatter_tensor(shard, full_grad, group=self.process_group)
                if self.gradient_postdivide_factor > 1:
                    shard.div_(self.gradient_postdivide_factor)
            if shard.dtype != self.flat_param.dtype:
                if stream is not None:
                    with torch.cuda.stream(stream):
                        shard = shard.to(self.flat_param.dtype)
                else:
                    shard = shard.to(self.flat_param.dtype)
            self._accumulate_shard_grad(shard, owns_buffer=False)
        if self.world_size > 1:
            # the reduced slice now lives in ``flat_param.grad``; the next micro-batch of the same update
            # (``--update-freq`` > 1) must overwrite the flat buffer, not add to what was already reduced
            for v in self._views:
                if hasattr(v, "_grad_filled"):
                    v._grad_filled = False
        if self.reshard_after_forward:
            self._free_full()

    def _collect_view_grads(self):
        """Gradients that autograd accumulated on the views (modular path) are folded into the
        flat gradient buffer; gradients the kernels wrote directly are already there."""
        if self._full_grad is None:
            return
        for v in self._views:
            g = v.grad
            gv = getattr(v, "_grad_view", None)
            if g is not None and gv is not None:
                if getattr(v, "_grad_filled", False):
                    gv.add_(g.to(gv.dtype))
                else:
                    gv.copy_(g)
                    v._grad_filled = True
                v.grad = None

    def _accumulate_shard_grad(self, shard: torch.Tensor, owns_buffer: bool):
        if shard.device != self.flat_param.device:
            side = getattr(self._root(), "_side_stream", None)
            if side is not None and shard.is_cuda:
                torch.cuda.current_stream().wait_stream(side)
            shard = shard[: self.flat_param.numel()].to(self.flat_param.device)  # offloaded: device -> host
            owns_buffer = False
        if self.flat_param.grad is None:
            self.flat_param.grad = shard if shard.numel() == self.flat_param.numel() else shard[: self.flat_param.numel()]
            if owns_buffer:
                # world size 1: the flat gradient buffer itself is the parameter's gradient; the
                # next backward must accumulate into it, so keep it and mark every view as filled.
                for v in self._views:
                    v._grad_filled = True
        elif self.flat_param.grad.data_ptr() != shard.data_ptr():
            side = getattr(self._root(), "_side_stream", None)
            if side is not None and shard.is_cuda:
                torch.cuda.current_stream().wait_stream(side)  # the shard is produced on the communication stream
            self.flat_param.grad.add_(shard)

    def _finish_backward(self):
        """End of the whole backward pass (root only): units whose input carried no gradient
        (e.g. the embedding) are reduced here, then compute waits for outstanding collectives."""
        for u in self._units:
            u._post_backward()
        comm = self.__dict__.get("_peer_comm")
        if self._reduce_pending and comm is not None and comm.pulls_gradients and self._side_stream is not None:
            # every rank has read what it needs of this rank's gradient buffers before the next backward may
            # overwrite them (with --update-freq > 1 no other collective sits in between)
            with torch.cuda.stream(self._side_stream):
                comm.barrier()
        if self._reduce_pending and self._side_stream is not None:
            torch.cuda.current_stream().wait_stream(self._side_stream)
        self._reduce_pending = False
        self._backward_armed = False

    # ------------------------------------------------------------- step hooks
    def zero_grad(self, set_to_none: bool = True):
        for u in (self._units if self._is_root else [self]):
            if u.flat_param is not None:
                u.flat_param.grad = None
            for v in u._views:
                v.grad = None
                if hasattr(v, "_grad_filled"):
                    v._grad_filled = False  # the next gradient written to the view overwrites

    def after_optimizer_step(self):
        """Local shards changed: every gathered copy is stale."""
        self._lazy_init()
        for u in self._units:
            if u.has_params and not u._aliases_shard():
                u._needs_gather = True
        self._step_gathered = False
        if self.__dict__.get("_peer_comm") is not None and not self.reshard_after_forward:
            # the shards are final: push them now, behind the optimizer kernels, instead of at the next forward
            self.prefetch_all()
            self._step_gathered = True

    # ------------------------------------------------------------ state dicts
    def _unit_paths(self) -> List[Tuple[str, "FullyShardedDataParallel"]]:
        out = []
        for name, m in self.named_modules():
            if isinstance(m, FullyShardedDataParallel):
                out.append((_clean_name(name), m))
        return out

    def local_state_dict(self, *args, **kwargs) -> Dict[str, torch.Tensor]:
        sd = {}
        for path, u in self._unit_paths():
            if u.flat_param is not None:
                key = f"{path}.flat_param_0" if path else "flat_param_0"
                t = u.flat_param.data
                sd[key] = t.cpu() if self.state_dict_device == torch.device("cpu") or self.state_dict_device == "cpu" else t
        for name, buf in self.named_buffers():
            sd[_clean_name(name)] = buf
        return sd

    def local_metadata_dict(self) -> Dict[str, Any]:
        param_metadata = []
        for path, u in self._unit_paths():
            if u.flat_param is None:
                continue
            param_metadata.append({
                "fsdp_path": path,
                "params": {
                    "flat_param_0": {
                        "names": list(u.param_names),
                        "shapes": [torch.Size(s) for s in u.param_shapes],
                        "numels": list(u.param_numels),
                        "padding": int(min(u.shard_numel, max(0, (u.rank + 1) * u.shard_numel - u.unpadded_numel))),
                    }
                },
                "no_broadcast_optim_state": False,
                "shared_param_info": list(u.shared_param_info),
            })
        return {"param_metadata": param_metadata, "buffer_names": [_clean_name(n) for n, _ in self.named_buffers()]}

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        """Unflattened parameters under their original names (collective over the group)."""
        sd = {}
        for path, u in self._unit_paths():
            if u.flat_param is None:
                continue
            had = u._full_param is not None and not u._needs_gather
            with torch.no_grad():
                u._gather_full()
                u._wait_gather()
            full = u._full_param
            off = 0
            for name, shape, n in zip(u.param_names, u.param_shapes, u.param_numels):
                key = f"{path}.{name}" if path else name
                sd[key] = full[off:off + n].view(shape).clone()
                off += n
            for shared_name, src_name in u.shared_param_info:
                k1 = f"{path}.{shared_name}" if path else shared_name
                k2 = f"{path}.{src_name}" if path else src_name
                sd[k1] = sd[k2]
            if not had and u.world_size > 1:
                u._free_full()
        for name, buf in self.named_buffers():
            sd[_clean_name(name)] = buf
        return sd

    def state_dict(self, *args, **kwargs):
        if self.use_sharded_state:
            return self.local_state_dict()
        full = self.full_state_dict()
        if self.rank == 0 or self.world_size == 1:
            return full
        return {}

    def load_local_state_dict(self, state_dict: Dict[str, torch.Tensor], strict: bool = True):
        missing = []
        for path, u in self._unit_paths():
            if u.flat_param is None:
                continue
            key = f"{path}.flat_param_0" if path else "flat_param_0"
            if key not in state_dict:
                missing.append(key)
                continue
            src = state_dict[key]
            n = min(src.numel(), u.flat_param.numel())
            with torch.no_grad():
                u.flat_param.data[:n].copy_(src.reshape(-1)[:n])
                if n < u.flat_param.numel():
                    u.flat_param.data[n:].zero_()
            u._needs_gather = True
        bufs = dict(self.named_buffers())
        for name, buf in bufs.items():
            k = _clean_name(name)
            if k in state_dict:
                buf.data.copy_(state_dict[k])
        if strict and missing:
            raise KeyError(f"missing keys in sharded state dict: {missing}")
        self._lazy_init()
        self._step_gathered = False

    def load_full_state_dict(self, state_dict: Dict[str, torch.Tensor], strict: bool = True):
        for path, u in self._unit_paths():
            if u.flat_param is None:
                continue
            flat = torch.zeros(u.padded_numel, dtype=u.flat_param.dtype)
            off = 0
            for name, shape, n in zip(u.param_names, u.param_shapes, u.param_numels):
                key = f"{path}.{name}" if path else name
                if key in state_dict:
                    flat[off:off + n].copy_(state_dict[key].reshape(-1))
                elif strict:
                    raise KeyError(f"missing key {key}")
                off += n
            with torch.no_grad():
                u.flat_param.data.copy_(flat[u.rank * u.shard_numel:(u.rank + 1) * u.shard_numel])
            u._needs_gather = True
        for name, buf in self.named_buffers():
            k = _clean_name(name)
            if k in state_dict:
                buf.data.copy_(state_dict[k])
        self._lazy_init()
        self._step_gathered = False

    def load_state_dict(self, state_dict, strict: bool = True, model_cfg=None):
        if any(k.endswith("flat_param_0") for k in state_dict):
            return self.load_local_state_dict(state_dict, strict)
        return self.load_full_state_dict(state_dict, strict)

    # ---------------------------------------------------------------- helpers
    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)

    @contextlib.contextmanager
    def summon_full_params(self):
        self._lazy_init()
        units = self._units
        with torch.no_grad():
            for u in units:
                u._gather_full()
                u._wait_gather()
        try:
            yield
        finally:
            for u in units:
                if u.world_size > 1:
                    u._free_full()

    @property
    def is_fsdp(self):
        return True


def _map_first_tensor(out, fn):
    if torch.is_tensor(out):
        return fn(out)
    if isinstance(out, tuple) and len(out) > 0 and torch.is_tensor(out[0]):
        return (fn(out[0]),) + tuple(out[1:])
    return out


def _clean_name(name: str) -> str:
    parts = [p for p in name.split(".") if p not in ("module", "_fsdp_wrapped_module", "_fpw_module", "")]
    return ".".join(parts)


# --------------------------------------------------------------------- wrap API
_WRAP_KWARGS: Optional[Dict[str, Any]] = None


@contextlib.contextmanager
def fsdp_enable_wrap(cfg_dist, use_sharded_state: bool = False, **kwargs):
    """Inside this context ``fsdp_wrap(module)`` wraps; outside it returns the module unchanged.
    Maps the distributed-training config onto wrapper arguments the way the reference does
    (metaseq/distributed/fully_sharded_data_parallel.py:85-124)."""
    global _WRAP_KWARGS
    if getattr(cfg_dist, "ddp_backend", None) != "fully_sharded":
        yield
        return
    group = kwargs.pop("process_group", None)
    if os.environ.get("RESHARD_OVERRIDE_PROCESS_GROUP", "False") == "True":
        group = DummyProcessGroup(rank=0, size=1)
    elif group is None:
        from . import utils as dist_utils

        group = dist_utils.get_data_parallel_group()
    compute_dtype = torch.bfloat16 if getattr(cfg_dist, "bf16", False) else (
        torch.float16 if getattr(cfg_dist, "fp16", False) else torch.float32)
    prev = _WRAP_KWARGS
    _WRAP_KWARGS = {
        "process_group": group,
        "reshard_after_forward": not getattr(cfg_dist, "no_reshard_after_forward", False),
        "mixed_precision": bool(getattr(cfg_dist, "fp16", False)) and not getattr(cfg_dist, "memory_efficient_fp16", False),
        "fp32_reduce_scatter": getattr(cfg_dist, "fp32_reduce_scatter", False),
        "flatten_parameters": True,
        "cpu_offload": getattr(cfg_dist, "cpu_offload", False),
        "compute_dtype": compute_dtype,
        "bucket_cap_mb": getattr(cfg_dist, "bucket_cap_mb", 25),
        "state_dict_device": torch.device("cpu"),
        "gradient_predivide_factor": getattr(cfg_dist, "gradient_predivide_factor", None),
        "use_sharded_state": use_sharded_state,
        "comm": getattr(cfg_dist, "comm_backend", None),
        **kwargs,
    }
    try:
        yield
    finally:
        _WRAP_KWARGS = prev


def fsdp_wrap(module: nn.Module, min_num_params: Optional[int] = None, **kwargs) -> nn.Module:
    """Wraps ``module`` when called inside ``fsdp_enable_wrap`` (and, if ``min_num_params`` is
    given, only when the module has at least that many parameters)."""
    if _WRAP_KWARGS is None:
        return module
    if min_num_params is not None:
        n = sum(p.numel() for p in module.parameters())
        if n < min_num_params:
            return module
    kw = dict(_WRAP_KWARGS)
    kw.update(kwargs)
    return FullyShardedDataParallel(module, **kw)
