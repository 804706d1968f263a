"""Raw (non-autograd) operator entry points.

Every function has two implementations with the same contract:

* the sm_100a kernel from ``libmsq_kernels.so`` when the tensors are CUDA
  fp16/bf16 and the library is present;
* a plain PyTorch fp32-accumulating restatement used on CPU, as the numerical
  oracle in the tests, and as the ``torch`` baseline backend.

``set_backend("torch")`` forces the PyTorch path on a GPU too (that is the
cuBLAS + unfused-ops baseline the kernels are compared against).
"""
from __future__ import annotations

import logging
import math
import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib

_BACKEND = "auto"  # "auto" | "torch"


def set_backend(name: str):
    global _BACKEND
    if name not in ("auto", "kernels", "torch"):
        raise ValueError(name)
    _BACKEND = "auto" if name == "kernels" else name


def get_backend() -> str:
    return _BACKEND


_GEMM_VARIANT = os.environ.get("MSQ_GEMM_VARIANT", "auto")  # "auto" | "1cta" | "2cta"


def set_gemm_variant(name: str):
    """``1cta``: one CTA per 128x256 tile; ``2cta``: CTA pairs on 256x256 tiles (cta_group::2);
    ``auto``: pairs for problems with at least 256 rows."""
    global _GEMM_VARIANT
    if name not in ("auto", "1cta", "2cta"):
        raise ValueError(name)
    _GEMM_VARIANT = name


def use_kernels(*tensors) -> bool:
    if _BACKEND == "torch":
        return False
    t = tensors[0]
    if not t.is_cuda or t.dtype not in (torch.float16, torch.bfloat16):
        return False
    if not _lib.kernels_path().exists():
        raise RuntimeError(
            "CUDA tensors were passed to metaseq_b200.ops but libmsq_kernels.so is not built; "
            "run `python -m metaseq_b200.build_ext`"
        )
    return True


_STRICT = os.environ.get("MSQ_STRICT_KERNELS", "0") == "1"
_FALLBACKS_SEEN: set = set()


def set_strict_kernels(on: bool = True):
    """With strict kernels an operator that would leave the sm_100a kernel path on CUDA 16-bit inputs (unsupported
    head size, stride or alignment) raises instead of running the PyTorch restatement (``--strict-kernels``)."""
    global _STRICT
    _STRICT = bool(on)


def _note_fallback(op: str, why: str):
    """Called where CUDA 16-bit tensors miss a kernel's shape / layout conditions: logs the reason once per
    (operator, reason), or raises under ``set_strict_kernels``."""
    if _BACKEND == "torch":
        return
    if _STRICT:
        raise RuntimeError(f"{op}: no sm_100a kernel for this call ({why}) and strict kernels are on")
    key = (op, why)
    if key not in _FALLBACKS_SEEN:
        _FALLBACKS_SEEN.add(key)
        logging.getLogger(__name__).warning("%s runs on PyTorch ops, not on the sm_100a kernel: %s", op, why)


def _bf(t) -> int:
    return 1 if t.dtype == torch.bfloat16 else 0


# ----------------------------------------------------------------------- GEMM
def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    mask: Optional[torch.Tensor] = None,
    relu: bool = False,
    out: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    bn: int = 0,
    max_ctas: int = 0,
    b_ready=None,
    gelu: bool = False,
) -> torch.Tensor:
    """``out[M,N] = epilogue(op(a) @ op(b))`` for 2-D operands.

    ``b_ready`` (or an attribute ``_msq_ready`` on ``b``) names the arrival flags of a ``b`` that peer GPUs
    are still writing (a view of a gathered FSDP buffer): an object with ``ready_struct(b)`` returning the
    ``GemmReady`` descriptor and ``wait(b)`` blocking the stream; the 2-CTA kernel polls the flags per tile.

    ``a`` is stored ``[M,K]`` (``a_mn=False``) or ``[K,M]`` (``a_mn=True``);
    ``b`` is stored ``[N,K]`` (``b_mn=False``, an ``nn.Linear`` weight) or
    ``[K,N]`` (``b_mn=True``).  Epilogue order: ``+bias`` -> ReLU (or GELU with ``gelu``) ->
    zero where ``mask<=0`` -> ``+residual`` -> ``+out`` (when ``accumulate``).  GELU is an epilogue of the
    few-row kernel only; elsewhere it is applied by PyTorch after the product.
    Operands may be row-strided views (last dim contiguous).
    """
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"inner dims differ: {K} vs {Kb}"
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    if M == 0 or N == 0:
        return out
    if gelu:
        assert not relu and mask is None and not accumulate
        few_rows = (use_kernels(a) and M <= 64 and not a_mn and not b_mn and bn == 0 and max_ctas == 0
                    and _GEMM_VARIANT == "auto" and K % 8 == 0 and N % 8 == 0 and b_ready is None
                    and _gemm_operands_ok(a, b, out, residual, None)
                    and getattr(b, "_msq_ready", None) is None and getattr(a, "_msq_ready", None) is None)
        if not few_rows:
            gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, out=out, bn=bn, max_ctas=max_ctas, b_ready=b_ready)
            act = torch.nn.functional.gelu(out.float())
            out.copy_(act + residual.float() if residual is not None else act)
            return out
    if use_kernels(a) and K % 8 == 0 and N % 8 == 0 and _gemm_operands_ok(a, b, out, residual, mask) \
            and (bias is None or bias.data_ptr() % 16 == 0):
        lib = _lib.kernels()
        if M <= 64 and not a_mn and not b_mn and mask is None and not accumulate and bn == 0 and max_ctas == 0 \
                and _GEMM_VARIANT == "auto" and b_ready is None and getattr(b, "_msq_ready", None) is None \
                and getattr(a, "_msq_ready", None) is None and out.data_ptr() != (residual.data_ptr() if residual is not None else 0):
            # a few rows (a decode step): one pass over the weights, K split over a thread-block cluster
            rc = lib.msq_gemm_skinny(
                _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0), _bf(a),
                _lib.ptr(bias), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
                2 if gelu else int(relu), _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr())
            _lib.check_rc(rc, "msq_gemm_skinny")
            return out
        pair = _GEMM_VARIANT == "2cta" or (_GEMM_VARIANT == "auto" and M >= 256 and N >= 128 and bn == 0)
        # Operands that peers are still writing carry a handle.  The kernel can poll one operand: a weight used as B
        # (handle.operand == 0) or a row-gathered activation used as A (handle.operand == 1); anything else is
        # awaited on the stream before the launch.
        hb = b_ready if b_ready is not None else getattr(b, "_msq_ready", None)
        ha = getattr(a, "_msq_ready", None)
        b_ready, target = None, None
        if hb is not None:
            if getattr(hb, "operand", 0) == 0:
                b_ready, target = hb, b
            else:
                hb.wait(b)
        if ha is not None:
            if b_ready is None and getattr(ha, "operand", 0) == 1:
                b_ready, target = ha, a
            else:
                ha.wait(a)
        if b_ready is not None:
            desc = b_ready.ready_struct(target) if pair else None
            if desc is None:
                b_ready.wait(target)  # kernel variant without flag polling: block the stream instead
                b_ready = None
        if b_ready is not None:
            import ctypes as _ct

            rc = lib.msq_gemm2_ready(
                _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K,
                a.stride(0), b.stride(0), out.stride(0),
                int(a_mn), int(b_mn), _bf(a),
                _lib.ptr(bias), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
                _lib.ptr(mask), mask.stride(0) if mask is not None else 0,
                int(relu), int(accumulate), bn, max_ctas,
                _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr(), _ct.byref(desc),
            )
            _lib.check_rc(rc, "msq_gemm2_ready")
            return out
        fn = lib.msq_gemm2 if pair else lib.msq_gemm
        rc = fn(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K,
            a.stride(0), b.stride(0), out.stride(0),
            int(a_mn), int(b_mn), _bf(a),
            _lib.ptr(bias), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
            _lib.ptr(mask), mask.stride(0) if mask is not None else 0,
            int(relu), int(accumulate), bn, max_ctas,
            _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "msq_gemm")
        return out
    if a.is_cuda and a.dtype in (torch.float16, torch.bfloat16):
        _note_fallback("gemm", f"K={K} N={N} must be multiples of 8, operands 16-byte aligned with unit inner stride")
    ensure_operand_ready(a)
    ensure_operand_ready(b)
    return _gemm_torch(a, b, a_mn, b_mn, bias, residual, mask, relu, out, accumulate)


def gemm_with_row_stats(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """``a @ w^T (+ bias)`` for ``a`` ``[M, K]`` and an ``nn.Linear`` weight ``w`` ``[N, K]`` whose epilogue also leaves
    the softmax pieces of every row per 256-column tile: returns ``(out, (rs_max, rs_sum))`` with the two fp32
    ``[tiles_n, M]`` tables of the tile maxima and of ``sum(exp(x - max))`` over the values as stored, or
    ``(out, None)`` where the pair kernel does not apply (the caller then reads the logits instead)."""
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    ok = (use_kernels(a) and a.dtype == w.dtype and M >= 256 and N >= 128 and K % 8 == 0 and N % 8 == 0
          and _GEMM_VARIANT != "1cta" and _gemm_operands_ok(a, w, out, None, None)
          and (bias is None or bias.data_ptr() % 16 == 0) and hasattr(_lib.kernels()._lib, "msq_gemm2_rowstats"))
    if not ok:
        return gemm(a, w, bias=bias, out=out), None
    lib = _lib.kernels()
    desc = None
    hb, ha = getattr(w, "_msq_ready", None), getattr(a, "_msq_ready", None)
    if hb is not None:
        if getattr(hb, "operand", 0) == 0:
            desc = hb.ready_struct(w)
        if desc is None:
            hb.wait(w)
    if ha is not None:
        if desc is None and getattr(ha, "operand", 0) == 1:
            desc = ha.ready_struct(a)
            if desc is None:
                ha.wait(a)
        else:
            ha.wait(a)
    tiles_n = int(lib.msq_gemm2_tiles_n(N))
    stats = torch.empty((2, tiles_n, M), dtype=torch.float32, device=a.device)
    import ctypes as _ct

    rc = lib.msq_gemm2_rowstats(_lib.ptr(a), _lib.ptr(w), _lib.ptr(out), M, N, K, a.stride(0), w.stride(0), out.stride(0),
                                0, 0, _bf(a), _lib.ptr(bias), _lib.ptr(stats[0]), _lib.ptr(stats[1]), 0,
                                _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr(),
                                _ct.byref(desc) if desc is not None else None)
    _lib.check_rc(rc, "msq_gemm2_rowstats")
    return out, (stats[0], stats[1])


def ensure_operand_ready(t: torch.Tensor):
    """Blocks the current stream until ``t`` (a view of a gathered buffer that peers may still be filling)
    is complete.  No-op for ordinary tensors."""
    h = getattr(t, "_msq_ready", None)
    if h is not None:
        h.wait(t)


def _gemm_operands_ok(a, b, out, residual, mask) -> bool:
    for t in (a, b, out, residual, mask):  # 2-D operands
        if t is None:
            continue
        if t.stride(-1) != 1 or t.data_ptr() % 16 or (t.dim() == 2 and t.stride(0) % 8):
            return False
    return True


def _gemm_torch(a, b, a_mn, b_mn, bias, residual, mask, relu, out, accumulate):
    am = a.t() if a_mn else a
    bm = b if b_mn else b.t()
    if a.is_cuda:
        acc = torch.matmul(am, bm).float()  # cuBLAS, fp32 accumulate inside
    else:
        acc = torch.matmul(am.float(), bm.float())
    if bias is not None:
        acc = acc + bias.float()
    if relu:
        acc = torch.relu(acc)
    if mask is not None:
        acc = acc * (mask > 0)
    if residual is not None:
        acc = acc + residual.float()
    if accumulate:
        acc = acc + out.float()
    out.copy_(acc)
    return out


# -------------------------------------------------------------------- RMS norm
def rms_norm_fwd(x2d, gamma, eps: float):
    """``y = x * rsqrt(mean(x^2) + eps) * gamma``; returns ``(y, rstd)`` with fp32 ``rstd``."""
    rows, D = x2d.shape
    if use_kernels(x2d) and D % 8 == 0 and D <= 16384 and x2d.is_contiguous():
        y = torch.empty_like(x2d)
        rstd = torch.empty(rows, dtype=torch.float32, device=x2d.device)
        rc = _lib.kernels().msq_rmsnorm_fwd(_lib.ptr(x2d), _lib.ptr(gamma), _lib.ptr(y), _lib.ptr(rstd), rows, D,
                                            float(eps), _bf(x2d), _lib.stream_ptr())
        _lib.check_rc(rc, "msq_rmsnorm_fwd")
        return y, rstd
    xf = x2d.float()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=1) + eps)
    y = xf * rstd[:, None]
    if gamma is not None:
        y = y * gamma.float()
    return y.to(x2d.dtype), rstd


def rms_norm_bwd(dy, x2d, rstd, gamma):
    """Returns ``(dx, dgamma)`` (``dgamma`` is ``None`` without ``gamma``)."""
    rows, D = x2d.shape
    if use_kernels(x2d) and D % 8 == 0 and D <= 16384 and x2d.is_contiguous() and dy.is_contiguous():
        lib = _lib.kernels()
        dx = torch.empty_like(x2d)
        part_g = part_b = dgamma = None
        if gamma is not None:
            parts = lib.msq_layernorm_bwd_parts(rows)
            part = torch.empty((2, parts, D), dtype=torch.float32, device=x2d.device)
            part_g, part_b = part[0], part[1]
            dgamma = torch.empty(D, dtype=x2d.dtype, device=x2d.device)
        rc = lib.msq_rmsnorm_bwd(_lib.ptr(dy), _lib.ptr(x2d), _lib.ptr(rstd), _lib.ptr(gamma), None, _lib.ptr(dx),
                                 _lib.ptr(part_g), _lib.ptr(part_b), _lib.ptr(dgamma), 0, rows, D, _bf(x2d),
                                 _lib.stream_ptr())
        _lib.check_rc(rc, "msq_rmsnorm_bwd")
        return dx, dgamma
    xf, dyf = x2d.float(), dy.float()
    xhat = xf * rstd[:, None]
    gdy = dyf * gamma.float() if gamma is not None else dyf
    dx = rstd[:, None] * (gdy - xhat * (gdy * xhat).mean(dim=1, keepdim=True))
    dg = (dyf * xhat).sum(dim=0).to(x2d.dtype) if gamma is not None else None
    return dx.to(x2d.dtype), dg


# ------------------------------------------------------------------ LayerNorm
def layer_norm_fwd(x2d, gamma, beta, eps: float):
    """Returns ``(y, mean, rstd)`` for ``x2d`` of shape ``[rows, D]``; statistics are fp32."""
    rows, D = x2d.shape
    if use_kernels(x2d) and D % 8 == 0 and D <= 16384 and x2d.is_contiguous():
        y = torch.empty_like(x2d)
        mean = torch.empty(rows, dtype=torch.float32, device=x2d.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x2d.device)
        rc = _lib.kernels().msq_layernorm_fwd(
            _lib.ptr(x2d), _lib.ptr(gamma), _lib.ptr(beta), _lib.ptr(y), _lib.ptr(mean), _lib.ptr(rstd),
            rows, D, float(eps), _bf(x2d), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "msq_layernorm_fwd")
        return y, mean, rstd
    if x2d.is_cuda and x2d.dtype in (torch.float16, torch.bfloat16):
        _note_fallback("layer_norm", f"width {D} must be a multiple of 8 and at most 16384, rows contiguous")
    xf = x2d.float()
    mean = xf.mean(dim=1)
    var = xf.var(dim=1, unbiased=False)
    rstd = torch.rsqrt(var + eps)
    y = (xf - mean[:, None]) * rstd[:, None]
    if gamma is not None:
        y = y * gamma.float()
    if beta is not None:
        y = y + beta.float()
    return y.to(x2d.dtype), mean, rstd


def layer_norm_bwd(dy, x2d, mean, rstd, gamma, add=None, dgamma_out=None, dbeta_out=None, accumulate=False,
                   need_param_grads=True):
    """Returns ``(dx, dgamma, dbeta)``.  ``add`` (same shape as ``x2d``) is summed into ``dx``:
    it carries the residual-branch gradient so no separate add kernel is needed."""
    rows, D = x2d.shape
    affine = gamma is not None and need_param_grads
    if use_kernels(x2d) and D % 8 == 0 and D <= 16384 and x2d.is_contiguous() and dy.is_contiguous():
        lib = _lib.kernels()
        dx = torch.empty_like(x2d)
        part_g = part_b = None
        if affine:
            parts = lib.msq_layernorm_bwd_parts(rows)
            part = torch.empty((2, parts, D), dtype=torch.float32, device=x2d.device)
            part_g, part_b = part[0], part[1]
            if dgamma_out is None:
                dgamma_out = torch.empty(D, dtype=x2d.dtype, device=x2d.device)
                dbeta_out = torch.empty(D, dtype=x2d.dtype, device=x2d.device)
                accumulate = False
        rc = lib.msq_layernorm_bwd(
            _lib.ptr(dy), _lib.ptr(x2d), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(gamma), _lib.ptr(add),
            _lib.ptr(dx), _lib.ptr(part_g), _lib.ptr(part_b),
            _lib.ptr(dgamma_out if affine else None), _lib.ptr(dbeta_out if affine else None),
            int(accumulate), rows, D, _bf(x2d), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "msq_layernorm_bwd")
        return dx, (dgamma_out if affine else None), (dbeta_out if affine else None)
    xf, dyf = x2d.float(), dy.float()
    xhat = (xf - mean[:, None]) * rstd[:, None]
    gdy = dyf * gamma.float() if gamma is not None else dyf
    m1 = gdy.mean(dim=1, keepdim=True)
    m2 = (gdy * xhat).mean(dim=1, keepdim=True)
    dx = rstd[:, None] * (gdy - m1 - xhat * m2)
    if add is not None:
        dx = dx + add.float()
    dg = db = None
    if affine:
        dg = (dyf * xhat).sum(dim=0)
        db = dyf.sum(dim=0)
        if dgamma_out is not None:
            if accumulate:
                dgamma_out.add_(dg.to(dgamma_out.dtype))
                dbeta_out.add_(db.to(dbeta_out.dtype))
            else:
                dgamma_out.copy_(dg)
                dbeta_out.copy_(db)
            dg, db = dgamma_out, dbeta_out
        else:
            dg, db = dg.to(x2d.dtype), db.to(x2d.dtype)
    return dx.to(x2d.dtype), dg, db


# ------------------------------------------------------------------ attention
def attn_keep_mask_reference(B: int, H: int, T: int, p: float, seed: int, device) -> torch.Tensor:
    """``[B, H, T, T]`` keep mask of the attention-dropout kernels, recomputed with integer tensor ops."""
    thr = int(p * 65536.0 + 0.5)
    rows = torch.arange(B * H * T, device=device, dtype=torch.int64).view(B, H, T, 1)
    kcol = torch.arange(T, device=device, dtype=torch.int64).view(1, 1, 1, T)
    pair = rows * ((T + 1) >> 1) + (kcol >> 1)

    def h32(x):
        x = x & 0xFFFFFFFF
        x = x ^ (x >> 16)
        x = (x * 0x7FEB352D) & 0xFFFFFFFF
        x = x ^ (x >> 15)
        x = (x * 0x846CA68B) & 0xFFFFFFFF
        return x ^ (x >> 16)

    hi = h32((pair >> 32) ^ ((seed >> 32) & 0xFFFFFFFF))
    bits = h32((pair & 0xFFFFFFFF) ^ (seed & 0xFFFFFFFF) ^ hi)
    half = torch.where((kcol & 1) == 0, bits & 0xFFFF, bits >> 16)
    return half >= thr


_ATTN_HEAD_DIMS = "multiples of 8 up to 128"


def attn_head_dim_ok(d: int) -> bool:
    """Head sizes of the flash-attention kernels: 64 and 128 natively, other multiples of 8 up to 128 (80 and 96 of
    OPT-2.7B / OPT-760M) zero-padded inside the kernel."""
    return 8 <= d <= 128 and d % 8 == 0


def _mask_args(doc_start, alibi_slopes, B, T, H, device):
    """Device pointers for the optional per-token document starts (int32 ``[B, T]``) and per-head ALiBi slopes
    (fp32 ``[H]``); the tensors are returned too so that they outlive the launch."""
    ds = sl = None
    if doc_start is not None:
        ds = doc_start.to(device=device, dtype=torch.int32).contiguous()
        assert ds.shape == (B, T), (ds.shape, B, T)
    if alibi_slopes is not None:
        sl = alibi_slopes.to(device=device, dtype=torch.float32).contiguous()
        assert sl.numel() == H
    return ds, sl


def flash_attn_fwd(q, k, v, scale: float, causal: bool = True, dropout_p: float = 0.0, seed: int = 0,
                   doc_start=None, alibi_slopes=None):
    """``q, k, v``: ``[B, T, H, d]`` views (last dim contiguous, head stride ``d``).
    Returns ``(out [B, T, H*d], lse [B, H, T] fp32)``.  With ``dropout_p > 0`` the attention weights are dropped
    with the mask derived from ``seed`` (the normaliser is unaffected); pass the same values to the backward.
    ``doc_start`` (``[B, T]``, the first position of each token's document) restricts a query to the keys of its own
    document; ``alibi_slopes`` (``[H]``) adds ``slope * key position`` to the scaled scores."""
    B, T, H, d = q.shape
    if use_kernels(q) and attn_head_dim_ok(d) and _attn_views_ok(q, k, v) and (doc_start is None or causal):
        out = torch.empty((B, T, H * d), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
        ds, sl = _mask_args(doc_start, alibi_slopes, B, T, H, q.device)
        rc = _lib.kernels().msq_flash_fwd(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v),
            q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0),
            _lib.ptr(out), out.stride(1), out.stride(0), _lib.ptr(lse),
            B, T, H, d, float(scale), int(causal), _bf(q), _lib.ptr(ds), _lib.ptr(sl), float(dropout_p), int(seed),
            _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "msq_flash_fwd")
        return out, lse
    if q.is_cuda and q.dtype in (torch.float16, torch.bfloat16):
        _note_fallback("flash_attn_fwd", f"head size {d} (kernels: {_ATTN_HEAD_DIMS}) or q/k/v views not 16-byte "
                                         "aligned [B,T,H,d] slices; this path materialises [B,H,T,T] scores")
    return _attn_fwd_torch(q, k, v, scale, causal, dropout_p, seed, doc_start, alibi_slopes)


def _attn_views_ok(*ts) -> bool:
    for t in ts:
        d = t.shape[-1]
        if t.stride(3) != 1 or t.stride(2) != d or t.data_ptr() % 16 or t.stride(1) % 8 or t.stride(0) % 8:
            return False
    return True


def _attn_scores_torch(qf, kf, scale, causal, doc_start, alibi_slopes):
    """fp32 ``[B, H, T, T]`` scores with every mask applied (the oracle of the kernels' masking)."""
    T = qf.shape[2]
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    pos = torch.arange(T, device=qf.device)
    if alibi_slopes is not None:
        s = s + alibi_slopes.to(s.device).float().view(1, -1, 1, 1) * pos.view(1, 1, 1, T).float()
    if causal:
        s = s.masked_fill((pos[None, :] > pos[:, None])[None, None], float("-inf"))
    if doc_start is not None:
        before_doc = pos.view(1, 1, T) < doc_start.to(s.device).long().view(-1, T, 1)  # [B, Tq, Tk]
        s = s.masked_fill(before_doc[:, None], float("-inf"))
    return s


def _attn_fwd_torch(q, k, v, scale, causal, dropout_p: float = 0.0, seed: int = 0, doc_start=None, alibi_slopes=None):
    B, T, H, d = q.shape
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))  # [B,H,T,d]
    s = _attn_scores_torch(qf, kf, scale, causal, doc_start, alibi_slopes)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    if dropout_p > 0:
        keep = attn_keep_mask_reference(B, H, T, dropout_p, seed, q.device)
        p = torch.where(keep, p / (1.0 - int(dropout_p * 65536.0 + 0.5) / 65536.0), torch.zeros_like(p))
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).reshape(B, T, H * d)
    return o.to(q.dtype), lse


def flash_attn_bwd(q, k, v, out, d_out, lse, scale: float, causal: bool, dq, dk, dv, dropout_p: float = 0.0,
                   seed: int = 0, doc_start=None, alibi_slopes=None):
    """Writes gradients into the ``[B, T, H, d]`` views ``dq, dk, dv`` (typically column slices
    of the qkv-gradient buffer).  Masks and dropout as given to the forward call."""
    B, T, H, d = q.shape
    if (
        use_kernels(q) and attn_head_dim_ok(d) and _attn_views_ok(q, k, v, dk, dv)
        and out.stride() == d_out.stride() and out.stride(2) == 1 and (doc_start is None or causal)
    ):
        delta = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
        dq_acc = torch.zeros((B, T, H * d), dtype=torch.float32, device=q.device)
        ds, sl = _mask_args(doc_start, alibi_slopes, B, T, H, q.device)
        rc = _lib.kernels().msq_flash_bwd(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(d_out),
            q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0),
            out.stride(1), out.stride(0), d_out.stride(1), d_out.stride(0),
            _lib.ptr(lse), _lib.ptr(delta), _lib.ptr(dq_acc), _lib.ptr(dk), _lib.ptr(dv),
            dk.stride(1), dk.stride(0), dv.stride(1), dv.stride(0),
            B, T, H, d, float(scale), int(causal), _bf(q), _lib.ptr(ds), _lib.ptr(sl), float(dropout_p), int(seed),
            _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "msq_flash_bwd")
        # dq is a column slice of the qkv gradient: rows of H*d elements, row stride dq.stride(1)
        if dq.stride(2) == d and dq.stride(3) == 1 and dq.stride(0) == T * dq.stride(1) and dq.stride(1) % 8 == 0:
            rc = _lib.kernels().msq_convert_rows(_lib.ptr(dq_acc), _lib.ptr(dq), B * T, H * d, dq.stride(1), _bf(dq),
                                                 _lib.stream_ptr())
            _lib.check_rc(rc, "msq_convert_rows")
        else:
            dq.copy_(dq_acc.view(B, T, H, d))
        return
    if q.is_cuda and q.dtype in (torch.float16, torch.bfloat16):
        _note_fallback("flash_attn_bwd", f"head size {d} (kernels: {_ATTN_HEAD_DIMS}) or views not 16-byte aligned "
                                         "[B,T,H,d] slices; this path materialises [B,H,T,T] scores")
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    of = out.float().view(B, T, H, d).permute(0, 2, 1, 3)
    dof = d_out.float().reshape(B, T, H, d).permute(0, 2, 1, 3)
    s = _attn_scores_torch(qf, kf, scale, causal, doc_start, alibi_slopes)
    p = torch.exp(s - lse[..., None])
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    if dropout_p > 0:
        keep = attn_keep_mask_reference(B, H, T, dropout_p, seed, q.device)
        ks = keep.float() / (1.0 - int(dropout_p * 65536.0 + 0.5) / 65536.0)
        dvf = torch.matmul((p * ks).transpose(-1, -2), dof)
        dp = dp * ks
    else:
        dvf = torch.matmul(p.transpose(-1, -2), dof)
    delta = (dof * of).sum(dim=-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dqf = torch.matmul(ds, kf)
    dkf = torch.matmul(ds.transpose(-1, -2), qf)
    dq.copy_(dqf.permute(0, 2, 1, 3))
    dk.copy_(dkf.permute(0, 2, 1, 3))
    dv.copy_(dvf.permute(0, 2, 1, 3))


# ------------------------------------------------------------------ embedding
def embed_fwd(tokens, positions, tok_w, pos_w, scale: float, vocab_start: int = 0, vocab_end: Optional[int] = None,
              add_positions: bool = True):
    """``out[r] = tok_w[tokens[r]-vocab_start]*scale (0 outside the partition) + pos_w[positions[r]]``."""
    D = tok_w.shape[1]
    if vocab_end is None:
        vocab_end = vocab_start + tok_w.shape[0]
    flat_tok = tokens.reshape(-1)
    flat_pos = positions.reshape(-1) if positions is not None else None
    rows = flat_tok.numel()
    use_pos = bool(add_positions and pos_w is not None and positions is not None)
    if use_kernels(tok_w) and D % 8 == 0:
        out = torch.empty((rows, D), dtype=tok_w.dtype, device=tok_w.device)
        # keep the contiguous copies alive until after the launch: two temporaries created inside the
        # argument list would be freed one after the other and end up at the same address
        tok_c = flat_tok.contiguous()
        pos_c = flat_pos.contiguous() if use_pos else None
        rc = _lib.kernels().msq_embed_fwd(
            _lib.ptr(tok_c), _lib.ptr(pos_c),
            _lib.ptr(tok_w), _lib.ptr(pos_w if use_pos else None), _lib.ptr(out),
            rows, D, float(scale), int(vocab_start), int(vocab_end), int(use_pos), _bf(tok_w), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "msq_embed_fwd")
        return out.view(*tokens.shape, D)
    in_range = (flat_tok >= vocab_start) & (flat_tok < vocab_end)
    idx = (flat_tok - vocab_start).clamp(0, tok_w.shape[0] - 1)
    out = tok_w[idx].float() * scale * in_range[:, None]
    if use_pos:
        out = out + pos_w[flat_pos].float()
    return out.to(tok_w.dtype).view(*tokens.shape, D)


def embed_bwd(tokens, positions, dy, tok_rows: int, pos_rows: int, scale: float, pad_idx: int,
              vocab_start: int = 0, need_pos: bool = True):
    """Returns fp32 gradient tables ``(dtok [tok_rows, D], dpos [pos_rows, D] or None)``."""
    D = dy.shape[-1]
    flat_tok = tokens.reshape(-1).contiguous()
    flat_pos = positions.reshape(-1).contiguous() if (positions is not None and need_pos) else None
    dy2 = dy.reshape(-1, D)
    vocab_end = vocab_start + tok_rows
    dtok = torch.zeros((tok_rows, D), dtype=torch.float32, device=dy.device)
    dpos = torch.zeros((pos_rows, D), dtype=torch.float32, device=dy.device) if flat_pos is not None else None
    if use_kernels(dy2) and D % 2 == 0 and dy2.is_contiguous():
        rc = _lib.kernels().msq_embed_bwd(
            _lib.ptr(flat_tok), _lib.ptr(flat_pos), _lib.ptr(dy2), _lib.ptr(dtok), _lib.ptr(dpos),
            dy2.shape[0], D, float(scale), int(vocab_start), int(vocab_end), int(pad_idx), _bf(dy2),
            _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "msq_embed_bwd")
        return dtok, dpos
    dyf = dy2.float()
    ok = (flat_tok >= vocab_start) & (flat_tok < vocab_end) & (flat_tok != pad_idx)
    idx = (flat_tok - vocab_start).clamp(0, tok_rows - 1)
    dtok.index_add_(0, idx, dyf * scale * ok[:, None])
    if dpos is not None:
        okp = flat_pos != pad_idx
        dpos.index_add_(0, flat_pos, dyf * okp[:, None])
    return dtok, dpos


def fold_fp32_into(src32: torch.Tensor, dst16: torch.Tensor, accumulate: bool):
    """``dst16 (+)= src32`` elementwise, with the sum formed in fp32."""
    n = src32.numel()
    if use_kernels(dst16) and n % 2 == 0 and dst16.is_contiguous() and src32.is_contiguous():
        rc = _lib.kernels().msq_fold_fp32(_lib.ptr(src32), _lib.ptr(dst16), n, int(accumulate), _bf(dst16),
                                          _lib.stream_ptr())
        _lib.check_rc(rc, "msq_fold_fp32")
        return dst16
    if accumulate:
        dst16.copy_(dst16.float() + src32.view_as(dst16))
    else:
        dst16.copy_(src32.view_as(dst16))
    return dst16


def _keep_mask_reference(rows: int, cols: int, p: float, seed: int, device) -> torch.Tensor:
    """The kernels' keep mask recomputed with integer tensor ops (oracle for tests and the PyTorch backend)."""
    thr = int(p * 65536.0 + 0.5)
    idx = torch.arange(rows * cols, device=device, dtype=torch.int64)
    pair = idx >> 1

    def h32(x):
        x = x & 0xFFFFFFFF
        x = x ^ (x >> 16)
        x = (x * 0x7FEB352D) & 0xFFFFFFFF
        x = x ^ (x >> 15)
        x = (x * 0x846CA68B) & 0xFFFFFFFF
        return x ^ (x >> 16)

    hi = h32((pair >> 32) ^ ((seed >> 32) & 0xFFFFFFFF))
    bits = h32((pair & 0xFFFFFFFF) ^ (seed & 0xFFFFFFFF) ^ hi)
    half = torch.where((idx & 1) == 0, bits & 0xFFFF, bits >> 16)
    return (half >= thr).view(rows, cols)


def dropout_add(y: torch.Tensor, bias, residual, p: float, seed: int, out: Optional[torch.Tensor] = None):
    """``residual + dropout(y + bias, p)`` for 2-D ``y`` with the mask derived from ``seed`` (same mask for the
    same seed, so the backward pass calls this again on the gradient with ``bias = residual = None``)."""
    rows, cols = y.shape
    if out is None:
        out = torch.empty_like(y)
    thr = int(p * 65536.0 + 0.5)
    if use_kernels(y) and cols % 8 == 0 and y.stride(1) == 1 and out.stride(1) == 1 and y.stride(0) % 8 == 0 \
            and out.stride(0) % 8 == 0 and (residual is None or (residual.stride(1) == 1 and residual.stride(0) % 8 == 0)):
        rc = _lib.kernels().msq_dropout_add(_lib.ptr(y), y.stride(0), _lib.ptr(bias), _lib.ptr(residual),
                                            residual.stride(0) if residual is not None else 0, _lib.ptr(out), out.stride(0),
                                            rows, cols, float(p), int(seed), _bf(y), _lib.stream_ptr())
        _lib.check_rc(rc, "msq_dropout_add")
        return out
    keep = _keep_mask_reference(rows, cols, p, seed, y.device)
    v = y.float() + (bias.float() if bias is not None else 0.0)
    v = torch.where(keep, v / (1.0 - thr / 65536.0), torch.zeros_like(v))
    if residual is not None:
        v = v + residual.float()
    out.copy_(v.to(out.dtype))
    return out


def decode_head_dim_ok(d: int) -> bool:
    """Head sizes of the decode-attention kernels (others than 64 and 128 run zero-padded lanes)."""
    return 8 <= d <= 128 and d % 8 == 0


def _decode_pad(d: int) -> int:
    return 64 if d <= 64 else 128


def decode_attn(q, k_cache, v_cache, length: int, num_heads: int, scale: float, key_padding_mask=None):
    """Single-query attention for incremental decoding.

    ``q``: ``[B, 1, H*d]`` (or ``[B, H*d]``); ``k_cache`` / ``v_cache``: ``[B, Tmax, H*d]`` of which the first
    ``length`` positions are valid (the new token's key/value already appended); ``key_padding_mask``:
    optional ``[B, >=length]`` bool / uint8, non-zero = excluded.  Returns ``[B, 1, H*d]``."""
    B = q.shape[0]
    D = q.shape[-1]
    d = D // num_heads
    q2 = q.reshape(B, D)
    if use_kernels(q) and decode_head_dim_ok(d) and q2.stride(-1) == 1 and k_cache.stride(-1) == 1 and v_cache.stride(-1) == 1 \
            and k_cache.stride() == v_cache.stride() and q2.data_ptr() % 16 == 0 and k_cache.data_ptr() % 16 == 0 \
            and v_cache.data_ptr() % 16 == 0 and q2.stride(0) % 8 == 0 and k_cache.stride(1) % 8 == 0:
        lib = _lib.kernels()
        out = torch.empty((B, D), dtype=q.dtype, device=q.device)
        splits = lib.msq_decode_attn_splits(B, num_heads, length)
        ws = torch.empty((B * num_heads * splits * (_decode_pad(d) + 2),), dtype=torch.float32, device=q.device) \
            if splits > 1 else None
        mask_c = None
        if key_padding_mask is not None:
            mask_c = key_padding_mask.to(torch.uint8)
            if mask_c.stride(-1) != 1:
                mask_c = mask_c.contiguous()
        rc = lib.msq_decode_attn(_lib.ptr(q2), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(out), _lib.ptr(mask_c),
                                 B, num_heads, d, length, q2.stride(0), k_cache.stride(1), k_cache.stride(0), out.stride(0),
                                 mask_c.stride(0) if mask_c is not None else 0, float(scale), _bf(q), _lib.ptr(ws), splits,
                                 _lib.stream_ptr())
        _lib.check_rc(rc, "msq_decode_attn")
        return out.view(B, 1, D)
    if q.is_cuda and q.dtype in (torch.float16, torch.bfloat16):
        _note_fallback("decode_attn", f"head size {d} (kernels: {_ATTN_HEAD_DIMS}) or cache layout")
    k = k_cache[:, :length].reshape(B, length, num_heads, d).transpose(1, 2).float()
    v = v_cache[:, :length].reshape(B, length, num_heads, d).transpose(1, 2).float()
    qh = q2.reshape(B, num_heads, 1, d).float() * scale
    scores = torch.matmul(qh, k.transpose(-1, -2))
    if key_padding_mask is not None:
        scores = scores.masked_fill(key_padding_mask[:, None, None, :length].bool(), float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, v).transpose(1, 2).reshape(B, 1, D).to(q.dtype)


class dependent_launch:
    """Context in which the few-row GEMM, the LayerNorm forward and the decode attention are launched with
    programmatic dependent launch: each kernel may start while its predecessor drains, and the GEMM requests its
    first weight tiles before waiting for it.  Valid only where the ``b`` operands of those GEMMs are not
    written by kernels in flight (a decode step, where they are the model weights)."""

    def __enter__(self):
        self._lib = _lib.kernels() if torch.cuda.is_available() and get_backend() != "torch" else None
        if self._lib is not None:
            self._lib.msq_set_dependent_launch(1)
        return self

    def __exit__(self, *exc):
        if self._lib is not None:
            self._lib.msq_set_dependent_launch(0)
        return False


def decode_attn_step(q, k_new, v_new, k_cache, v_cache, length_dev, num_heads: int, scale: float, length_hint: int):
    """One decode step with the cache length held on the device (usable inside a CUDA graph).

    ``q`` / ``k_new`` / ``v_new``: ``[B, H*d]`` row views (last dim contiguous, equal batch strides for the two
    new rows); ``k_cache`` / ``v_cache``: ``[B, Tmax, H*d]``; ``length_dev``: int32 tensor with the number of
    cached positions.  The new key/value become position ``length_dev`` of the cache and take part in the
    attention; the caller adds one to ``length_dev`` afterwards.  ``length_hint`` (host) sizes the sequence
    split only.  Kernel-only: there is no PyTorch restatement because the point is the absence of host state."""
    B, D = q.shape
    d = D // num_heads
    assert k_new.stride(0) == v_new.stride(0) and k_cache.stride() == v_cache.stride()
    lib = _lib.kernels()
    out = torch.empty((B, D), dtype=q.dtype, device=q.device)
    splits = lib.msq_decode_attn_splits(B, num_heads, max(1, length_hint))
    ws = torch.empty((B * num_heads * splits * (_decode_pad(d) + 2),), dtype=torch.float32, device=q.device) \
        if splits > 1 else None
    rc = lib.msq_decode_attn_step(_lib.ptr(q), _lib.ptr(k_new), _lib.ptr(v_new), k_new.stride(0), _lib.ptr(k_cache),
                                  _lib.ptr(v_cache), _lib.ptr(out), None, B, num_heads, d, _lib.ptr(length_dev),
                                  k_cache.shape[1], q.stride(0), k_cache.stride(1), k_cache.stride(0), out.stride(0), 0,
                                  float(scale), _bf(q), _lib.ptr(ws), splits, _lib.stream_ptr())
    _lib.check_rc(rc, "msq_decode_attn_step")
    return out


# -------------------------------------------------------------- cross entropy
def cross_entropy_fwd_bwd(logits2d, target, ignore_index: int, grad_scale: float, write_grad: bool):
    """Per-row NLL (fp32, 0 where ``target == ignore_index``) and log-sum-exp.  With
    ``write_grad`` the logits buffer is overwritten by ``(softmax - onehot) * grad_scale``."""
    rows, V = logits2d.shape
    if use_kernels(logits2d) and V % 8 == 0 and V * 2 <= 200 * 1024 and logits2d.stride(1) == 1 \
            and logits2d.stride(0) % 8 == 0:
        loss = torch.empty(rows, dtype=torch.float32, device=logits2d.device)
        lse = torch.empty(rows, dtype=torch.float32, device=logits2d.device)
        target_c = target.contiguous()
        rc = _lib.kernels().msq_cross_entropy(
            _lib.ptr(logits2d), logits2d.stride(0), _lib.ptr(target_c), _lib.ptr(loss), _lib.ptr(lse),
            rows, V, int(ignore_index), float(grad_scale), int(write_grad), _bf(logits2d), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "msq_cross_entropy")
        return loss, lse
    if logits2d.is_cuda and logits2d.dtype in (torch.float16, torch.bfloat16):
        _note_fallback("cross_entropy", f"vocabulary {V} must be a multiple of 8 and at most 102400 per rank")
    lf = logits2d.float()
    lse = torch.logsumexp(lf, dim=1)
    valid = target != ignore_index
    tgt = target.clamp(0, V - 1)
    loss = (lse - lf.gather(1, tgt[:, None]).squeeze(1)) * valid
    if write_grad:
        g = torch.exp(lf - lse[:, None])
        g.scatter_add_(1, tgt[:, None], -torch.ones_like(lse)[:, None])
        g = g * (valid[:, None] * grad_scale)
        logits2d.copy_(g)
    return loss, lse


def cross_entropy_from_row_stats(logits2d, target, ignore_index: int, grad_scale: float, row_stats):
    """Per-row NLL for logits whose producing GEMM left ``row_stats = (rs_max, rs_sum)``; the logits are
    overwritten with ``(softmax - onehot) * grad_scale``.  One small kernel folds the tiles of each row, one pass
    over the logits writes the gradient."""
    rows, V = logits2d.shape
    rs_max, rs_sum = row_stats
    tiles_n = rs_max.shape[0]
    assert rs_max.shape[1] == rows and logits2d.stride(1) == 1
    lib = _lib.kernels()
    tgt = target.contiguous()
    stats = torch.empty((1, rows, 3), dtype=torch.float32, device=logits2d.device)
    rc = lib.msq_ce_merge_rowstats(_lib.ptr(rs_max), _lib.ptr(rs_sum), tiles_n, rows, _lib.ptr(logits2d),
                                   logits2d.stride(0), _lib.ptr(tgt), V, 0, _lib.ptr(stats), None, 1, 0, rows, 0,
                                   _bf(logits2d), _lib.stream_ptr())
    _lib.check_rc(rc, "msq_ce_merge_rowstats")
    loss = torch.empty(rows, dtype=torch.float32, device=logits2d.device)
    rc = lib.msq_vp_ce_finish(_lib.ptr(logits2d), logits2d.stride(0), _lib.ptr(tgt), _lib.ptr(stats), 1, _lib.ptr(loss),
                              rows, V, 0, int(ignore_index), float(grad_scale), _bf(logits2d), _lib.stream_ptr())
    _lib.check_rc(rc, "msq_vp_ce_finish")
    return loss


def scale_rows_(x2d, g, ref: float = 1.0):
    """``x2d[r, :] *= g[r] / ref`` in place (``g`` with one element scales everything); ``g`` stays on the device.
    Used to apply the incoming gradient (the loss scale) to a gradient stored by the forward pass.  ``ref`` is the
    factor the stored values were already multiplied by: rows whose ``g`` equals it are not touched, so a forward
    pass that guessed the upstream factor makes this a launch of a few microseconds."""
    rows, cols = x2d.shape
    g = g.reshape(-1)
    assert g.numel() in (1, rows)
    kernel_ok = use_kernels(x2d) and cols % 8 == 0 and x2d.stride(1) == 1 and x2d.stride(0) % 8 == 0 \
        and x2d.data_ptr() % 16 == 0 and g.dtype in (torch.float32, x2d.dtype) and g.is_cuda
    if ref != 1.0:
        if kernel_ok and hasattr(_lib.kernels()._lib, "msq_scale_rows_rel"):
            g = g.contiguous()
            rc = _lib.kernels().msq_scale_rows_rel(_lib.ptr(x2d), x2d.stride(0), rows, cols, _lib.ptr(g),
                                                   int(g.dtype == torch.float32), int(g.numel() > 1), 1.0 / float(ref),
                                                   _bf(x2d), _lib.stream_ptr())
            _lib.check_rc(rc, "msq_scale_rows_rel")
            return x2d
        g = g.float() / float(ref)
        return x2d.mul_(g.to(x2d.dtype).reshape(-1, 1) if g.numel() > 1 else g.to(x2d.dtype))
    if kernel_ok:
        g = g.contiguous()
        rc = _lib.kernels().msq_scale_rows(_lib.ptr(x2d), x2d.stride(0), rows, cols, _lib.ptr(g),
                                           int(g.dtype == torch.float32), int(g.numel() > 1), _bf(x2d), _lib.stream_ptr())
        _lib.check_rc(rc, "msq_scale_rows")
        return x2d
    return x2d.mul_(g.to(x2d.dtype).reshape(-1, 1) if g.numel() > 1 else g.to(x2d.dtype))


# ------------------------------------------------------------------- sampling
def sample_top_p(lprobs, top_p, uniform=None):
    """One token per row from the nucleus of mass ``top_p`` (a float, or a ``[rows]`` tensor) of fp32
    log-probabilities ``[rows, V]`` (``-inf`` = banned).  Returns ``(log-prob of the token, token)``.
    ``uniform``: optional ``[rows]`` numbers in [0, 1) (drawn from the torch generator otherwise)."""
    rows, V = lprobs.shape
    if uniform is None:
        uniform = torch.rand(rows, device=lprobs.device, dtype=torch.float32)
    per_row = torch.is_tensor(top_p) and top_p.numel() > 1
    if lprobs.is_cuda and _BACKEND != "torch" and _lib.kernels_path().exists() and lprobs.dtype == torch.float32 \
            and lprobs.stride(1) == 1 and V <= 56000:
        p_t = top_p.to(device=lprobs.device, dtype=torch.float32).contiguous() if torch.is_tensor(top_p) else \
            torch.full((1,), float(top_p), device=lprobs.device, dtype=torch.float32)
        tok = torch.empty(rows, dtype=torch.long, device=lprobs.device)
        lp = torch.empty(rows, dtype=torch.float32, device=lprobs.device)
        rc = _lib.kernels().msq_sample_topp(_lib.ptr(lprobs), lprobs.stride(0), rows, V, _lib.ptr(p_t), int(per_row),
                                            _lib.ptr(uniform.contiguous()), _lib.ptr(tok), _lib.ptr(lp), _lib.stream_ptr())
        _lib.check_rc(rc, "msq_sample_topp")
        return lp, tok
    # the same draw in PyTorch: nucleus = {p >= threshold}, taken in index order
    probs = torch.exp(lprobs.float())
    probs = torch.where(torch.isfinite(probs), probs, torch.zeros_like(probs))
    sprobs, _ = probs.sort(descending=True, dim=-1)
    csum = sprobs.cumsum(dim=-1)
    p = top_p.to(lprobs.device).float().reshape(-1, 1) if torch.is_tensor(top_p) else float(top_p)
    keep_sorted = (csum - sprobs) < p  # always keeps the top token
    last = keep_sorted.long().sum(dim=-1, keepdim=True).clamp(min=1) - 1
    thr = sprobs.gather(-1, last)
    kept = torch.where((probs >= thr) & (probs > 0), probs, torch.zeros_like(probs))
    cdf = kept.cumsum(dim=-1)
    draw = uniform.to(lprobs.device).float().clamp(0, 0.99999994).reshape(-1, 1) * cdf[:, -1:]
    tok = (cdf <= draw).long().sum(dim=-1).clamp(max=V - 1)
    return lprobs.gather(-1, tok[:, None]).squeeze(-1), tok


# --------------------------------------------------------------------- colsum
_COLSUM_SCRATCH: dict = {}


def colsum(x2d, out16=None, accumulate=False):
    """Column sums of ``[rows, N]`` (bias gradient), fp32 accumulation."""
    rows, N = x2d.shape
    if out16 is not None and use_kernels(x2d) and N % 8 == 0 and x2d.stride(1) == 1 and x2d.stride(0) % 8 == 0 \
            and out16.is_contiguous() and out16.dtype == x2d.dtype:
        # one launch: partial sums by fp32 atomics into a persistent scratch that the kernel itself turns into the
        # 16-bit result and leaves zeroed (one scratch per device, stream and width)
        key = (x2d.device.index or 0, torch.cuda.current_stream(x2d.device).cuda_stream, N)
        scratch = _COLSUM_SCRATCH.get(key)
        if scratch is None:
            scratch = (torch.zeros(N, dtype=torch.float32, device=x2d.device),
                       torch.zeros((N + 255) // 256, dtype=torch.int32, device=x2d.device))
            _COLSUM_SCRATCH[key] = scratch
        rc = _lib.kernels().msq_colsum_direct(_lib.ptr(x2d), x2d.stride(0), rows, N, _lib.ptr(scratch[0]),
                                              _lib.ptr(scratch[1]), _lib.ptr(out16), int(accumulate), _bf(x2d),
                                              _lib.stream_ptr())
        _lib.check_rc(rc, "msq_colsum_direct")
        return out16
    if use_kernels(x2d) and N % 8 == 0 and x2d.stride(1) == 1 and x2d.stride(0) % 8 == 0:
        acc = torch.zeros(N, dtype=torch.float32, device=x2d.device)
        rc = _lib.kernels().msq_colsum(_lib.ptr(x2d), x2d.stride(0), rows, N, _lib.ptr(acc), _bf(x2d),
                                       _lib.stream_ptr())
        _lib.check_rc(rc, "msq_colsum")
    else:
        acc = x2d.float().sum(dim=0)
    if out16 is None:
        return acc.to(x2d.dtype)
    return fold_fp32_into(acc, out16, accumulate)


# ------------------------------------------------------------------ optimizer
def sumsq(g: torch.Tensor, out: torch.Tensor, accumulate: bool):
    """``out[0] (+)= sum(g**2)`` in fp32; ``out`` is a 1-element fp32 tensor on ``g``'s device."""
    n = g.numel()
    if g.is_cuda and _BACKEND != "torch" and g.is_contiguous() and _lib.kernels_path().exists():
        lib = _lib.kernels()
        parts = lib.msq_sumsq_parts(n)
        scratch = torch.empty(parts, dtype=torch.float32, device=g.device)
        rc = lib.msq_sumsq(_lib.ptr(g), n, _lib.dtype_code(g.dtype), _lib.ptr(scratch), _lib.ptr(out),
                           int(accumulate), _lib.stream_ptr())
        _lib.check_rc(rc, "msq_sumsq")
        return out
    s = g.float().pow(2).sum()
    if accumulate:
        out.add_(s)
    else:
        out.fill_(0).add_(s)
    return out


_SUMSQ_TABLES: dict = {}


def _tensor_table(tensors):
    """Device table {pointer, elements, first block} (+ scratch, ticket) that the list-form kernels walk; cached per
    device and stream and rebuilt only when a pointer or size changes."""
    t0 = tensors[0]
    dev = t0.device
    key = tuple((t.data_ptr(), t.numel()) for t in tensors)
    slot = (dev.index or 0, torch.cuda.current_stream(dev).cuda_stream)
    cached = _SUMSQ_TABLES.get(slot)
    if cached is None or cached[0] != key:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        total_n = sum(n for _, n in key)
        budget = 8 * sms  # blocks over all tensors, shared in proportion to their sizes (at least one each)
        per_block = 8 * 512
        recs, first = [], 0
        for ptr, n in key:
            want = max(1, min((n + per_block - 1) // per_block, max(1, round(budget * n / max(total_n, 1)))))
            recs.append((ptr, n, first))
            first += want
        recs.append((0, 0, first))
        table = torch.tensor([x for r in recs for x in r], dtype=torch.int64).to(dev)
        scratch = torch.empty(first, dtype=torch.float32, device=dev)
        ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        if len(_SUMSQ_TABLES) > 16:
            _SUMSQ_TABLES.clear()
        cached = (key, table, scratch, ticket, first)
        _SUMSQ_TABLES[slot] = cached
    return cached[1:]


def list_kernels_ok(tensors) -> bool:
    """True when the list-form kernels take ``tensors``: contiguous CUDA tensors of one 16/32-bit float type."""
    if not tensors or _BACKEND == "torch" or not tensors[0].is_cuda or not _lib.kernels_path().exists():
        return False
    dt = tensors[0].dtype
    return dt in (torch.float16, torch.bfloat16, torch.float32) and \
        all(t.dtype == dt and t.is_contiguous() and t.is_cuda for t in tensors)


def sumsq_multi(tensors, out: torch.Tensor, accumulate: bool):
    """``out[0] (+)= sum over all tensors of sum(t**2)`` in one launch (contiguous CUDA tensors of one dtype)."""
    table, scratch, ticket, total_blocks = _tensor_table(tensors)
    rc = _lib.kernels().msq_sumsq_multi(_lib.ptr(table), len(tensors), total_blocks, _lib.dtype_code(tensors[0].dtype),
                                        _lib.ptr(scratch), _lib.ptr(ticket), _lib.ptr(out), int(accumulate),
                                        _lib.stream_ptr())
    _lib.check_rc(rc, "msq_sumsq_multi")
    return out


def absmax_multi(tensors, out: torch.Tensor, accumulate: bool = False):
    """``out[0] = max |element|`` over the list in one launch (the inf-norm; +inf if any element is not finite)."""
    table, scratch, ticket, total_blocks = _tensor_table(tensors)
    rc = _lib.kernels().msq_absmax_multi(_lib.ptr(table), len(tensors), total_blocks,
                                         _lib.dtype_code(tensors[0].dtype), _lib.ptr(scratch), _lib.ptr(ticket),
                                         _lib.ptr(out), int(accumulate), _lib.stream_ptr())
    _lib.check_rc(rc, "msq_absmax_multi")
    return out


def scale_multi_(tensors, dev_scale: Optional[torch.Tensor] = None, host_scale: float = 1.0):
    """Every tensor of the list ``*= host_scale * dev_scale[0]`` in place, in one launch; ``dev_scale`` is a 1-element
    fp32 device tensor (e.g. a clip coefficient that never visits the host)."""
    table, _, _, total_blocks = _tensor_table(tensors)
    rc = _lib.kernels().msq_scale_multi(_lib.ptr(table), len(tensors), total_blocks,
                                        _lib.dtype_code(tensors[0].dtype),
                                        _lib.ptr(dev_scale) if dev_scale is not None else None, float(host_scale),
                                        _lib.stream_ptr())
    _lib.check_rc(rc, "msq_scale_multi")
    return tensors


def clip_decision(sumsq_terms: torch.Tensor, pre_factor: float, max_norm: float, ctrl: torch.Tensor):
    """Fills ``ctrl`` (4 fp32): [grad multiplier, skip flag, grad norm, clip coefficient]."""
    if sumsq_terms.is_cuda and _BACKEND != "torch" and _lib.kernels_path().exists():
        rc = _lib.kernels().msq_clip_decision(_lib.ptr(sumsq_terms), sumsq_terms.numel(), float(pre_factor),
                                              float(max_norm), _lib.ptr(ctrl), _lib.stream_ptr())
        _lib.check_rc(rc, "msq_clip_decision")
        return ctrl
    norm = pre_factor * torch.sqrt(sumsq_terms.float().sum())
    bad = not bool(torch.isfinite(norm))
    coef = 1.0
    if not bad and max_norm > 0:
        coef = min(1.0, max_norm / (float(norm) + 1e-6))
    ctrl[0] = pre_factor * coef
    ctrl[1] = 1.0 if bad else 0.0
    ctrl[2] = norm
    ctrl[3] = coef
    return ctrl


_ADAM_TABLES: dict = {}


def adamw_step_multi(items, *, lr, beta1, beta2, eps, weight_decay, step, ctrl=None):
    """One launch of the AdamW update over a list of ``(p, g, m, v)`` tensors that share data types,
    hyper-parameters and step count (the reference's ``multi_tensor_adam``).  The table of pointers lives on the
    device and is rebuilt only when a pointer or size changes.  Callers check eligibility (contiguous CUDA
    tensors, kernel backend)."""
    p0, g0 = items[0][0], items[0][1]
    key = tuple((p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel()) for p, g, m, v in items)
    dev_key = (p0.device.index or 0, len(items), key[0][0])
    cached = _ADAM_TABLES.get(dev_key)
    if cached is None or cached[0] != key:
        flat = [x for rec in key for x in rec]
        table = torch.tensor(flat, dtype=torch.int64).to(p0.device, non_blocking=False)
        if len(_ADAM_TABLES) > 32:
            _ADAM_TABLES.clear()
        cached = (key, table)
        _ADAM_TABLES[dev_key] = cached
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    step_size = lr * math.sqrt(bc2) / bc1
    rc = _lib.kernels().msq_adamw_multi(
        _lib.ptr(cached[1]), len(items), max(rec[4] for rec in key), _lib.dtype_code(p0.dtype), _lib.dtype_code(g0.dtype),
        float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), float(step_size), _lib.ptr(ctrl),
        _lib.stream_ptr())
    _lib.check_rc(rc, "msq_adamw_multi")


def adamw_step(p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step, ctrl=None, p16_out=None):
    """One AdamW update of a flat tensor (decoupled decay, bias correction folded into the
    step size, eps outside the sqrt).  ``ctrl`` is the device control block from
    ``clip_decision``: grads are multiplied by ``ctrl[0]`` and the whole update is a no-op
    when ``ctrl[1] != 0``."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    step_size = lr * math.sqrt(bc2) / bc1
    n = p.numel()
    if p.is_cuda and _BACKEND != "torch" and _lib.kernels_path().exists() and p.is_contiguous() and g.is_contiguous():
        rc = _lib.kernels().msq_adamw(
            _lib.ptr(p), _lib.ptr(g), _lib.ptr(m), _lib.ptr(v), _lib.ptr(p16_out),
            1 if (p16_out is not None and p16_out.dtype == torch.bfloat16) else 0,
            n, _lib.dtype_code(p.dtype), _lib.dtype_code(g.dtype),
            float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), float(step_size),
            _lib.ptr(ctrl), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "msq_adamw")
        return
    gmul = 1.0
    if ctrl is not None:
        if float(ctrl[1]) != 0.0:
            return
        gmul = float(ctrl[0])
    gf = g.float() * gmul
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    pf = p.float()
    pf = pf - lr * weight_decay * pf
    pf = pf - step_size * (m / (v.sqrt() + eps))
    p.copy_(pf)
    if p16_out is not None:
        p16_out.copy_(pf)
