"""ctypes loader for the in-tree native libraries.

The CUDA kernels live in ``metaseq_b200/_C/libmsq_kernels.so`` (built by
``metaseq_b200.build_ext``) and export a C ABI that takes raw device pointers
and a ``cudaStream_t``.  On a machine with a GPU the library must be present:
falling back silently to PyTorch ops there would hide a broken build, so
``kernels()`` raises instead.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

_ROOT = Path(__file__).resolve().parent.parent / "_C"
_KLIB = None
_HLIB = None

P = c_void_p
I = c_int
L = c_longlong
F = c_float


# kernels launched by one call of each entry point (used for the launch counter)
_KERNELS_PER_CALL = {"msq_flash_head_dim_ok": 0, "msq_symm_alloc": 0, "msq_symm_open": 0, "msq_symm_close": 0, "msq_symm_free": 0, "msq_sumsq": 2, "msq_layernorm_bwd": 2, "msq_rmsnorm_bwd": 2, "msq_flash_bwd": 2, "msq_layernorm_bwd_parts": 0,
                     "msq_sumsq_parts": 0, "msq_gemm2_tiles_n": 0, "msq_gemm_skinny_split": 0, "msq_set_dependent_launch": 0, "msq_gemm_skinny_set_prof": 0, "msq_decode_attn_splits": 0}
_LAUNCHES = [0]


def reset_launch_count():
    _LAUNCHES[0] = 0


def launch_count() -> int:
    """Number of kernels of this library launched since the last reset."""
    return _LAUNCHES[0]


class _Counted:
    """ctypes function wrapper that adds the entry point's kernel count to the launch counter."""

    __slots__ = ("fn", "n")

    def __init__(self, fn, n):
        self.fn, self.n = fn, n

    def __call__(self, *args):
        _LAUNCHES[0] += self.n
        return self.fn(*args)


class _CountingLib:
    def __init__(self, lib):
        self._lib = lib
        self._cache = {}

    def __getattr__(self, name):
        c = self._cache.get(name)
        if c is None:
            c = _Counted(getattr(self._lib, name), _KERNELS_PER_CALL.get(name, 1))
            self._cache[name] = c
        return c


def _sig(lib, name, argtypes, restype=c_int):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


class GemmReady(ctypes.Structure):
    """Arrival-flag description of a GEMM operand that lives in a gathered buffer (``MsqGemmReady`` in
    csrc/gemm2_sm100.cu)."""

    _fields_ = [("flags", c_void_p), ("b_offset", c_longlong), ("shard_bytes", c_longlong),
                ("chunk_bytes", c_longlong), ("chunks_per_shard", c_int), ("skip_shard", c_int),
                ("epoch", ctypes.c_uint), ("operand", c_int)]


def _declare_kernels(lib):
    _sig(lib, "msq_gemm", [P, P, P, I, I, I, L, L, L, I, I, I, P, P, L, P, L, I, I, I, I, P, P])
    if hasattr(lib, "msq_gemm2"):
        _sig(lib, "msq_gemm2", [P, P, P, I, I, I, L, L, L, I, I, I, P, P, L, P, L, I, I, I, I, P, P])
        _sig(lib, "msq_gemm2_ready", [P, P, P, I, I, I, L, L, L, I, I, I, P, P, L, P, L, I, I, I, I, P, P, P])
    _sig(lib, "msq_layernorm_bwd_parts", [I])
    _sig(lib, "msq_layernorm_fwd", [P, P, P, P, P, P, I, I, F, I, P])
    _sig(lib, "msq_layernorm_bwd", [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P])
    _sig(lib, "msq_sumsq_parts", [L])
    _sig(lib, "msq_sumsq", [P, L, I, P, P, I, P])
    _sig(lib, "msq_clip_decision", [P, I, F, F, P, P])
    _sig(lib, "msq_adamw", [P, P, P, P, P, I, L, I, I, F, F, F, F, F, F, P, P])
    _sig(lib, "msq_embed_fwd", [P, P, P, P, P, I, I, F, L, L, I, I, P])
    _sig(lib, "msq_embed_bwd", [P, P, P, P, P, I, I, F, L, L, L, I, P])
    _sig(lib, "msq_fold_fp32", [P, P, L, I, I, P])
    _sig(lib, "msq_convert_rows", [P, P, L, I, L, I, P])
    U = ctypes.c_uint
    _sig(lib, "msq_symm_alloc", [L, P, P])
    _sig(lib, "msq_symm_open", [P, P])
    _sig(lib, "msq_symm_close", [P])
    _sig(lib, "msq_symm_free", [P])
    _sig(lib, "msq_comm_barrier", [P, I, I, L, U, P, P])
    _sig(lib, "msq_comm_wait_flags", [P, L, L, L, L, U, P, P])
    _sig(lib, "msq_comm_wait_flag_list", [P, P, I, U, P, P])
    _sig(lib, "msq_comm_allgather_push", [P, L, P, L, I, I, I, P, L, U, I, P, P])
    _sig(lib, "msq_comm_reduce_scatter_push", [P, L, P, L, I, I, P, L, U, P, I, P, P])
    _sig(lib, "msq_comm_signal", [P, I, I, L, U, P])
    _sig(lib, "msq_comm_reduce_rows", [P, L, I, I, I, P, P, L, P, L, P, L, L, I, I, I, P, L, U, P, L, P, I, P, P])
    _sig(lib, "msq_gemm2_scatter", [P, P, I, I, I, L, L, L, I, I, I, P, I, I, I, P, P])
    _sig(lib, "msq_comm_allgather_ce", [P, L, P, L, I, I, I, P, L, U, P, P])
    _sig(lib, "msq_comm_reduce_scatter_ce", [P, L, P, L, I, I, P, L, U, P])
    _sig(lib, "msq_comm_reduce_slots", [P, L, I, F, P, I, I, P, P, P, L, U, I, P, P])
    _sig(lib, "msq_comm_allreduce_oneshot", [P, L, L, P, P, L, I, I, I, P, L, U, P, P])
    _sig(lib, "msq_comm_allreduce_sliced", [P, L, L, P, P, L, L, I, I, I, P, L, U, P, P])
    _sig(lib, "msq_comm_allreduce_multimem_fused", [P, P, P, P, L, L, I, I, I, P, L, U, P, P])
    _sig(lib, "msq_comm_allreduce_multimem", [P, L, I, I, I, P, L, U, I, P, P])
    _sig(lib, "msq_cross_entropy", [P, L, P, P, P, I, I, L, F, I, I, P])
    _sig(lib, "msq_colsum", [P, L, I, I, P, I, P])
    ULL = ctypes.c_ulonglong
    _sig(lib, "msq_flash_fwd", [P, P, P, L, L, L, L, L, L, P, L, L, P, I, I, I, I, F, I, I, P, P, F, ULL, P, P])
    _sig(
        lib,
        "msq_flash_bwd",
        [P, P, P, P, P] + [L] * 10 + [P, P, P, P, P] + [L] * 4 + [I, I, I, I, F, I, I, P, P, F, ULL, P, P],
    )
    _sig(lib, "msq_flash_head_dim_ok", [I])
    for name, sig in _OPTIONAL.items():
        if hasattr(lib, name):
            _sig(lib, name, sig)


# Entry points added by later source files; declared when present.
_OPTIONAL = {
    "msq_decode_attn": [P, P, P, P, P, I, I, I, I, L, L, L, L, L, F, I, P, I, P],
    "msq_decode_attn_splits": [I, I, I],
    "msq_gemm_skinny": [P, P, P, I, I, I, L, L, L, I, P, P, L, I, P, P],
    "msq_gemm_skinny_split": [I, I],
    "msq_gemm_skinny_allreduce": [P, P, P, I, I, I, L, L, L, I, P, P, L, I, I, I, P, I, P, I, P, P],
    "msq_set_dependent_launch": [I],
    "msq_gemm_skinny_set_prof": [P],
    "msq_scale_rows": [P, L, L, I, P, I, I, I, P],
    "msq_sample_topp": [P, L, I, I, P, I, P, P, P, P],
    "msq_adamw_multi": [P, I, L, I, I, F, F, F, F, F, F, P, P],
    "msq_rmsnorm_fwd": [P, P, P, P, I, I, F, I, P],
    "msq_rmsnorm_bwd": [P, P, P, P, P, P, P, P, P, I, I, I, I, P],
    "msq_decode_attn_step": [P, P, P, L, P, P, P, P, I, I, I, P, I, L, L, L, L, L, F, I, P, I, P],
    "msq_dropout_add": [P, L, P, P, L, P, L, L, I, F, ctypes.c_ulonglong, I, P],
    "msq_vp_ce_partial": [P, L, P, P, I, I, L, I, P],
    "msq_vp_ce_finish": [P, L, P, P, I, P, I, I, L, L, F, I, P],
    "msq_gemm2_tiles_n": [I],
    "msq_colsum_direct": [P, L, I, I, P, P, P, I, I, P],
    "msq_comm_words_exchange": [P, L, P, P, L, I, I, P, P, P, I, P, P],
    "msq_comm_reduce_scatter_pull": [P, P, L, L, I, I, F, P, I, I, P, P, P, L, ctypes.c_uint, I, P, P],
    "msq_comm_allgather_multimem": [P, P, L, I, I, I, P, L, ctypes.c_uint, I, P, P],
    "msq_sumsq_multi": [P, I, I, I, P, P, P, I, P],
    "msq_absmax_multi": [P, I, I, I, P, P, P, I, P],
    "msq_scale_multi": [P, I, I, I, P, F, P],
    "msq_gemm2_rowstats": [P, P, P, I, I, I, L, L, L, I, I, I, P, P, P, I, P, P, P],
    "msq_ce_merge_rowstats": [P, P, I, I, P, L, P, I, L, P, P, I, I, I, ctypes.c_uint, I, P],
    "msq_vp_ce_finish_exchanged": [P, L, P, P, I, I, ctypes.c_uint, P, I, I, L, L, F, I, P, P],
    "msq_scale_rows_rel": [P, L, L, I, P, I, I, F, I, P],
}
_OPTIONAL = {k: v for k, v in _OPTIONAL.items() if v is not None}


def kernels_path() -> Path:
    override = os.environ.get("MSQ_KERNELS_LIB")  # development aid: load an alternative build
    return Path(override) if override else _ROOT / "libmsq_kernels.so"


def host_path() -> Path:
    return _ROOT / "libmsq_host.so"


def have_kernels() -> bool:
    """True when the CUDA library is built and a GPU is present to run it."""
    return torch.cuda.is_available() and kernels_path().exists() and not os.environ.get("MSQ_DISABLE_KERNELS")


def kernels():
    """The CUDA kernel library (loaded on first use)."""
    global _KLIB
    if _KLIB is None:
        path = kernels_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: run `python -m metaseq_b200.build_ext` (or __graft_entry__.build()) first"
            )
        lib = ctypes.CDLL(str(path))
        _declare_kernels(lib)
        _KLIB = _CountingLib(lib)
    return _KLIB


def host():
    """The host-side C++ helper library, or None when it has not been built."""
    global _HLIB
    if _HLIB is None:
        path = host_path()
        if not path.exists():
            return None
        _HLIB = ctypes.CDLL(str(path))
    return _HLIB


def stream_ptr() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t) -> c_void_p:
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return 0
    if dt == torch.bfloat16:
        return 1
    if dt == torch.float32:
        return 2
    raise TypeError(f"unsupported dtype {dt}")


_STATUS = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels set when one of their bounded waits runs out."""
    key = torch.device(device).index or 0
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


_PEEK = {}


def peek_status(device="cuda") -> int:
    """Reads the status word without clearing it and without waiting for the work queued on the compute
    streams: the copy runs on a stream of its own into pinned memory.  For the host watchdog thread."""
    w = status_word(device)
    key = w.device.index or 0
    if key not in _PEEK:
        _PEEK[key] = (torch.cuda.Stream(device=w.device), torch.zeros(1, dtype=torch.int32).pin_memory())
    stream, host = _PEEK[key]
    with torch.cuda.stream(stream):
        host.copy_(w, non_blocking=True)
    stream.synchronize()
    return int(host[0])


def check_status(device="cuda") -> int:
    """Reads (and clears) the kernel status word; non-zero means a wait timed out."""
    w = status_word(device)
    v = int(w.item())
    if v:
        w.zero_()
    return v


def check_rc(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed to launch (code {rc})")
