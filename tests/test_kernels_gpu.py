"""Numerics of every sm_100a kernel against a plain PyTorch fp32 restatement of the same op.

The reference repository has no kernel-level tests for its vendored CUDA; these
fill that gap.  Inputs are 16-bit, the oracle accumulates in fp32 from the same
16-bit values, and outputs are compared after rounding to the output dtype.
"""
import math

import pytest
import torch

from metaseq_b200.ops import functional as F
from metaseq_b200.ops import _lib

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16]


def _tol(dtype):
    return (2e-2, 2e-2) if dtype == torch.bfloat16 else (4e-3, 4e-3)


def _close(got, want, dtype, scale=1.0):
    rtol, atol = _tol(dtype)
    torch.testing.assert_close(got.float(), want.float(), rtol=rtol, atol=atol * scale)


def _ref(fn, *args, **kw):
    prev = F.get_backend()
    F.set_backend("torch")
    try:
        return fn(*args, **kw)
    finally:
        F.set_backend(prev)


def _status_ok():
    assert _lib.check_status("cuda") == 0, "a kernel reported a timed-out wait"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 264, 136), (1024, 2048, 512), (384, 96, 1024)])
def test_gemm_layouts(dtype, a_mn, b_mn, M, N, K):
    torch.manual_seed(0)
    if a_mn and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0")
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=dtype)
    got = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    am = a.t() if a_mn else a
    bm = b if b_mn else b.t()
    want = am.float() @ bm.float()
    _status_ok()
    _close(got, want.to(dtype), dtype, scale=math.sqrt(K))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_epilogue(dtype, bn):
    torch.manual_seed(1)
    M, N, K = 520, 776, 320
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    w = torch.randn(N, K, device="cuda", dtype=dtype) * 0.05
    bias = torch.randn(N, device="cuda", dtype=dtype)
    res = torch.randn(M, N, device="cuda", dtype=dtype)
    mask = torch.randn(M, N, device="cuda", dtype=dtype)
    base = a.float() @ w.float().t()
    # bias + relu
    got = F.gemm(a, w, bias=bias, relu=True, bn=bn)
    _close(got, torch.relu(base + bias.float()).to(dtype), dtype)
    # bias + residual
    got = F.gemm(a, w, bias=bias, residual=res, bn=bn)
    _close(got, (base + bias.float() + res.float()).to(dtype), dtype)
    # mask (ReLU backward) and accumulate into an existing output
    prev = torch.randn(M, N, device="cuda", dtype=dtype)
    out = prev.clone()
    F.gemm(a, w, mask=mask, out=out, accumulate=True, bn=bn)
    _close(out, (base * (mask > 0) + prev.float()).to(dtype), dtype)
    _status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_strided_views(dtype):
    torch.manual_seed(2)
    M, K, N = 256, 128, 192
    big = torch.randn(M, 3 * K, device="cuda", dtype=dtype)
    a = big[:, K:2 * K]
    w = torch.randn(N, K, device="cuda", dtype=dtype)
    outbig = torch.zeros(M, 2 * N, device="cuda", dtype=dtype)
    F.gemm(a, w, out=outbig[:, N:])
    _close(outbig[:, N:], (a.float() @ w.float().t()).to(dtype), dtype, scale=math.sqrt(K))
    assert float(outbig[:, :N].abs().max()) == 0.0
    _status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [64, 2048, 4096, 7168])
@pytest.mark.parametrize("affine", [True, False])
def test_layernorm(dtype, D, affine):
    torch.manual_seed(3)
    rows = 777
    x = (torch.randn(rows, D, device="cuda") * 2 + 0.5).to(dtype)
    g = (torch.randn(D, device="cuda") * 0.2 + 1).to(dtype) if affine else None
    b = (torch.randn(D, device="cuda") * 0.2).to(dtype) if affine else None
    y, mean, rstd = F.layer_norm_fwd(x, g, b, 1e-5)
    yr, meanr, rstdr = _ref(F.layer_norm_fwd, x, g, b, 1e-5)
    _close(y, yr, dtype)
    torch.testing.assert_close(mean, meanr, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(rstd, rstdr, rtol=1e-4, atol=1e-4)
    dy = torch.randn(rows, D, device="cuda").to(dtype)
    add = torch.randn(rows, D, device="cuda").to(dtype)
    dx, dg, db = F.layer_norm_bwd(dy, x, mean, rstd, g, add=add)
    dxr, dgr, dbr = _ref(F.layer_norm_bwd, dy, x, mean, rstd, g, add=add)
    _close(dx, dxr, dtype)
    if affine:
        _close(dg, dgr, dtype, scale=math.sqrt(rows))
        _close(db, dbr, dtype, scale=math.sqrt(rows))


def _attn_inputs(B, T, H, d, dtype):
    qkv = (torch.randn(B, T, 3 * H * d, device="cuda") * 0.7).to(dtype)
    D = H * d
    k = qkv[..., 0:D].view(B, T, H, d)
    v = qkv[..., D:2 * D].view(B, T, H, d)
    q = qkv[..., 2 * D:].view(B, T, H, d)
    return qkv, q, k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("T", [128, 256, 200, 640])
def test_flash_attention_forward(dtype, d, T):
    torch.manual_seed(4)
    B, H = 2, 3
    _, q, k, v = _attn_inputs(B, T, H, d, dtype)
    scale = d ** -0.5
    out, lse = F.flash_attn_fwd(q, k, v, scale, True)
    outr, lser = _ref(F.flash_attn_fwd, q, k, v, scale, True)
    _status_ok()
    _close(out, outr, dtype)
    torch.testing.assert_close(lse, lser, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("T", [128, 384, 200])
def test_flash_attention_backward(dtype, d, T):
    torch.manual_seed(5)
    B, H = 2, 2
    qkv, q, k, v = _attn_inputs(B, T, H, d, dtype)
    D = H * d
    scale = d ** -0.5
    out, lse = _ref(F.flash_attn_fwd, q, k, v, scale, True)
    d_out = (torch.randn(B, T, D, device="cuda") * 0.5).to(dtype)

    def run(use_ref):
        dqkv = torch.zeros_like(qkv)
        dk = dqkv[..., 0:D].view(B, T, H, d)
        dv = dqkv[..., D:2 * D].view(B, T, H, d)
        dq = dqkv[..., 2 * D:].view(B, T, H, d)
        if use_ref:
            _ref(F.flash_attn_bwd, q, k, v, out, d_out, lse, scale, True, dq, dk, dv)
        else:
            F.flash_attn_bwd(q, k, v, out, d_out, lse, scale, True, dq, dk, dv)
        return dqkv

    got, want = run(False), run(True)
    _status_ok()
    _close(got, want, dtype, scale=4.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_cross_entropy(dtype):
    torch.manual_seed(6)
    rows, V = 300, 50272
    logits = (torch.randn(rows, V, device="cuda") * 3).to(dtype)
    target = torch.randint(0, V, (rows,), device="cuda")
    target[::7] = 1  # ignored (pad)
    l1 = logits.clone()
    loss, lse = F.cross_entropy_fwd_bwd(l1, target, 1, 128.0, True)
    l2 = logits.clone()
    lossr, lser = _ref(F.cross_entropy_fwd_bwd, l2, target, 1, 128.0, True)
    torch.testing.assert_close(loss, lossr, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(lse, lser, rtol=1e-3, atol=1e-3)
    _close(l1, l2, dtype, scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    torch.manual_seed(7)
    V, P, D, B, T = 1000, 70, 256, 3, 50
    tok_w = torch.randn(V, D, device="cuda").to(dtype)
    pos_w = torch.randn(P, D, device="cuda").to(dtype)
    tokens = torch.randint(0, V, (B, T), device="cuda")
    tokens[0, -5:] = 1
    positions = torch.randint(2, P, (B, T), device="cuda")
    positions[0, -5:] = 1
    out = F.embed_fwd(tokens, positions, tok_w, pos_w, 1.0)
    outr = _ref(F.embed_fwd, tokens, positions, tok_w, pos_w, 1.0)
    _close(out, outr, dtype)
    # vocab-parallel partition
    out = F.embed_fwd(tokens, positions, tok_w[500:], pos_w, 1.0, vocab_start=500, add_positions=False)
    outr = _ref(F.embed_fwd, tokens, positions, tok_w[500:], pos_w, 1.0, vocab_start=500, add_positions=False)
    _close(out, outr, dtype)
    dy = torch.randn(B, T, D, device="cuda").to(dtype)
    dt, dp = F.embed_bwd(tokens, positions, dy, V, P, 1.0, 1)
    dtr, dpr = _ref(F.embed_bwd, tokens, positions, dy, V, P, 1.0, 1)
    torch.testing.assert_close(dt, dtr, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(dp, dpr, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_colsum_and_fold(dtype):
    torch.manual_seed(8)
    x = torch.randn(3001, 776, device="cuda").to(dtype)
    got = F.colsum(x)
    _close(got, x.float().sum(0).to(dtype), dtype, scale=60.0)
    dst = torch.randn(776, device="cuda").to(dtype)
    want = (dst.float() + x.float().sum(0)).to(dtype)
    F.colsum(x, out16=dst, accumulate=True)
    _close(dst, want, dtype, scale=60.0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_sumsq_clip_adamw(dtype):
    torch.manual_seed(9)
    n = 1_000_003
    g = (torch.randn(n, device="cuda") * 3).to(dtype)
    acc = torch.zeros(2, dtype=torch.float32, device="cuda")
    F.sumsq(g, acc[0:1], False)
    F.sumsq(g[: n // 2], acc[1:2], False)
    want0 = g.float().pow(2).sum()
    torch.testing.assert_close(acc[0], want0, rtol=1e-4, atol=1e-2)
    ctrl = torch.zeros(4, dtype=torch.float32, device="cuda")
    F.clip_decision(acc, 1.0 / 128, 1.0, ctrl)
    norm = (acc.sum().sqrt() / 128).item()
    assert abs(ctrl[2].item() - norm) / norm < 1e-4
    assert ctrl[1].item() == 0.0
    assert abs(ctrl[0].item() - (1 / 128) * min(1.0, 1.0 / (norm + 1e-6))) < 1e-6
    # AdamW against the PyTorch restatement
    pdt = dtype
    p = torch.randn(n, device="cuda").to(pdt)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    p2, m2, v2 = p.clone(), m.clone(), v.clone()
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    for step in (1, 2):
        F.adamw_step(p, g, m, v, step=step, ctrl=ctrl, **kw)
        _ref(F.adamw_step, p2, g, m2, v2, step=step, ctrl=ctrl, **kw)
    torch.testing.assert_close(m, m2, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(v, v2, rtol=1e-4, atol=1e-8)
    torch.testing.assert_close(p.float(), p2.float(), rtol=1e-2 if pdt != torch.float32 else 1e-4, atol=1e-2 if pdt != torch.float32 else 1e-5)
    # overflow: non-finite norm sets the skip flag and the step leaves everything untouched
    acc[0] = float("inf")
    F.clip_decision(acc, 1.0, 1.0, ctrl)
    assert ctrl[1].item() == 1.0
    before = p.clone()
    F.adamw_step(p, g, m, v, step=3, ctrl=ctrl, **kw)
    assert torch.equal(before, p)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (1000, 264, 136), (2048, 2048, 1024), (384, 96 * 2, 512)])
def test_gemm_two_cta_layouts(dtype, a_mn, b_mn, M, N, K):
    """The cta_group::2 kernel (CTA pairs on 256x256 tiles) against fp32 matmul, all four layouts."""
    torch.manual_seed(10)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=dtype)
    F.set_gemm_variant("2cta")
    try:
        got = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    finally:
        F.set_gemm_variant("auto")
    am = a.t() if a_mn else a
    bm = b if b_mn else b.t()
    want = am.float() @ bm.float()
    _status_ok()
    _close(got, want.to(dtype), dtype, scale=math.sqrt(K))


@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_two_cta_epilogue(dtype):
    torch.manual_seed(12)
    M, N, K = 776, 520, 320
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    w = torch.randn(N, K, device="cuda", dtype=dtype) * 0.05
    bias = torch.randn(N, device="cuda", dtype=dtype)
    res = torch.randn(M, N, device="cuda", dtype=dtype)
    mask = torch.randn(M, N, device="cuda", dtype=dtype)
    base = a.float() @ w.float().t()
    F.set_gemm_variant("2cta")
    try:
        got = F.gemm(a, w, bias=bias, relu=True)
        _close(got, torch.relu(base + bias.float()).to(dtype), dtype)
        got = F.gemm(a, w, bias=bias, residual=res)
        _close(got, (base + bias.float() + res.float()).to(dtype), dtype)
        prev = torch.randn(M, N, device="cuda", dtype=dtype)
        out = prev.clone()
        F.gemm(a, w, mask=mask, out=out, accumulate=True)
        _close(out, (base * (mask > 0) + prev.float()).to(dtype), dtype)
    finally:
        F.set_gemm_variant("auto")
    _status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (4, 2048, 2048), (16, 6144, 2048), (17, 2048, 8192), (32, 8192, 2048),
                                   (33, 264, 136), (64, 50272, 768), (48, 96, 4096), (8, 1000, 200)])
@pytest.mark.parametrize("epilogue", ["plain", "bias_relu", "bias_residual", "bias_gelu"])
def test_gemm_few_rows_cluster_split_k(dtype, M, N, K, epilogue):
    """Products with at most 64 rows take the swapped-operand kernel whose K range is split over a cluster."""
    torch.manual_seed(M * 7 + N)
    x = torch.randn(M, K, device="cuda", dtype=dtype)
    w = torch.randn(N, K, device="cuda", dtype=dtype) * (K ** -0.5)
    bias = torch.randn(N, device="cuda", dtype=dtype) if epilogue != "plain" else None
    res = torch.randn(M, N, device="cuda", dtype=dtype) if epilogue == "bias_residual" else None
    relu = epilogue == "bias_relu"
    gelu = epilogue == "bias_gelu"
    split = _lib.kernels().msq_gemm_skinny_split(N, K)
    assert split in (1, 2, 4, 8)
    torch.cuda.synchronize()
    if (N, K) == (2048, 8192):
        assert split == 8
    before = _lib.launch_count()
    out = F.gemm(x, w, bias=bias, residual=res, relu=relu, gelu=gelu)
    assert _lib.launch_count() == before + 1
    ref = x.float() @ w.float().t()
    if bias is not None:
        ref = ref + bias.float()
    if relu:
        ref = torch.relu(ref)
    if gelu:
        ref = torch.nn.functional.gelu(ref)
    if res is not None:
        ref = ref + res.float()
    _close(out, ref, dtype)
    # row-strided input and output views
    big = torch.zeros(M, N + 16, device="cuda", dtype=dtype)
    xs = torch.randn(M, K + 8, device="cuda", dtype=dtype)
    xs[:, :K] = x
    F.gemm(xs[:, :K], w, bias=bias, residual=res, relu=relu, gelu=gelu, out=big[:, 8:8 + N])
    _close(big[:, 8:8 + N], ref, dtype)
    assert float(big[:, :8].abs().max()) == 0.0 and float(big[:, 8 + N:].abs().max()) == 0.0
    _status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("per_row,g_dtype", [(True, torch.float32), (False, torch.float32), (True, None), (False, None)])
def test_scale_rows_in_place(dtype, per_row, g_dtype):
    torch.manual_seed(5)
    rows, cols = 300, 1000
    buf = torch.randn(rows, cols + 24, device="cuda", dtype=dtype)
    view = buf[:, 8:8 + cols]
    g = torch.rand(rows if per_row else 1, device="cuda", dtype=g_dtype or dtype) * 4
    want = view.float() * (g.float().reshape(-1, 1) if per_row else g.float())
    untouched = buf.clone()
    before = _lib.launch_count()
    F.scale_rows_(view, g)
    assert _lib.launch_count() == before + 1
    _close(view, want, dtype)
    assert torch.equal(buf[:, :8], untouched[:, :8]) and torch.equal(buf[:, 8 + cols:], untouched[:, 8 + cols:])


def test_dependent_launch_chain_matches_ordinary_launches():
    """LayerNorm -> GEMM -> GEMM(+residual) chains launched with programmatic dependent launch (eagerly and from a
    CUDA graph) give the results of ordinary launches: each kernel waits for its predecessor before touching
    anything but the weights."""
    torch.manual_seed(3)
    dt = torch.float16
    x = torch.randn(32, 2048, device="cuda", dtype=dt)
    g, b = torch.randn(2048, device="cuda", dtype=dt), torch.randn(2048, device="cuda", dtype=dt)
    w1 = torch.randn(8192, 2048, device="cuda", dtype=dt) * 0.02
    w2 = torch.randn(2048, 8192, device="cuda", dtype=dt) * 0.02

    def chain(x):
        for _ in range(4):
            h, _, _ = F.layer_norm_fwd(x, g, b, 1e-5)
            f = F.gemm(h, w1, relu=True)
            x = F.gemm(f, w2, residual=x)
        return x

    want = chain(x)
    with F.dependent_launch():
        got = chain(x)
    assert torch.equal(got, want)
    xs = x.clone()
    with F.dependent_launch():
        chain(xs)  # warm-up outside capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = chain(xs)
    for _ in range(3):
        graph.replay()
    assert torch.equal(out, want)
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,d,S,Tmax", [(2, 4, 64, 37, 64), (16, 32, 64, 1000, 2050), (1, 8, 128, 2048, 2050), (3, 2, 128, 5, 8)])
@pytest.mark.parametrize("masked", [False, True])
def test_decode_attention_kv_cache(dtype, B, H, d, S, Tmax, masked):
    g = torch.Generator(device="cuda").manual_seed(B * 131 + S)
    D = H * d
    q = torch.randn(B, 1, D, device="cuda", dtype=dtype, generator=g)
    kc = torch.randn(B, Tmax, D, device="cuda", dtype=dtype, generator=g)
    vc = torch.randn(B, Tmax, D, device="cuda", dtype=dtype, generator=g)
    mask = None
    if masked:
        mask = torch.zeros(B, Tmax, dtype=torch.bool, device="cuda")
        for b in range(B):
            mask[b, : (b * 3) % max(1, S - 1)] = True  # left padding of different lengths
    out = F.decode_attn(q, kc, vc, S, H, d ** -0.5, mask)
    F.set_backend("torch")
    try:
        ref = F.decode_attn(q.float(), kc.float(), vc.float(), S, H, d ** -0.5, mask)
    finally:
        F.set_backend("auto")
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert torch.allclose(out.float(), ref.float(), rtol=tol, atol=tol), (out.float() - ref.float()).abs().max()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,d,S,Tmax", [(2, 4, 64, 37, 64), (16, 32, 64, 999, 1024), (1, 8, 128, 2047, 2050), (3, 2, 128, 0, 8)])
def test_decode_attention_step_appends_and_attends(dtype, B, H, d, S, Tmax):
    """Device-side length: the new key/value rows land at position ``S`` of the cache and the result equals
    attention over ``S + 1`` positions."""
    g = torch.Generator(device="cuda").manual_seed(B * 17 + S)
    D = H * d
    qkv = torch.randn(B, 3 * D, device="cuda", dtype=dtype, generator=g)
    kc = torch.randn(B, Tmax, D, device="cuda", dtype=dtype, generator=g)
    vc = torch.randn(B, Tmax, D, device="cuda", dtype=dtype, generator=g)
    k_ref, v_ref = kc.clone(), vc.clone()
    k_ref[:, S] = qkv[:, 0:D]
    v_ref[:, S] = qkv[:, D:2 * D]
    length = torch.tensor([S], dtype=torch.int32, device="cuda")
    out = F.decode_attn_step(qkv[:, 2 * D:], qkv[:, 0:D], qkv[:, D:2 * D], kc, vc, length, H, d ** -0.5, max(1, S))
    assert torch.equal(kc, k_ref) and torch.equal(vc, v_ref)
    F.set_backend("torch")
    try:
        ref = F.decode_attn(qkv[:, None, 2 * D:].float(), k_ref.float(), v_ref.float(), S + 1, H, d ** -0.5, None)
    finally:
        F.set_backend("auto")
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert torch.allclose(out.float(), ref[:, 0].float(), rtol=tol, atol=tol), (out.float() - ref[:, 0].float()).abs().max()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dropout_add_matches_hash_reference(dtype):
    g = torch.Generator(device="cuda").manual_seed(1)
    rows, cols = 777, 1024
    y = torch.randn(rows, cols, device="cuda", dtype=dtype, generator=g)
    bias = torch.randn(cols, device="cuda", dtype=dtype, generator=g)
    res = torch.randn(rows, cols + 64, device="cuda", dtype=dtype, generator=g)[:, :cols]  # strided rows
    out = F.dropout_add(y, bias, res, 0.1, 123456789012345)
    keep = F._keep_mask_reference(rows, cols, 0.1, 123456789012345, y.device)
    assert abs(keep.float().mean().item() - 0.9) < 5e-3
    ref = torch.where(keep, (y.float() + bias.float()) / (1 - 6554 / 65536), torch.zeros_like(y, dtype=torch.float32)) + res.float()
    tol = 3e-2 if dtype == torch.bfloat16 else 4e-3
    assert torch.allclose(out.float(), ref, rtol=tol, atol=tol)
    gout = F.dropout_add(y, None, None, 0.1, 123456789012345)  # backward form: same mask, no bias / residual
    assert torch.equal(gout == 0, ~keep | (y == 0))


@pytest.mark.parametrize("B,T,H,d", [(2, 256, 4, 64), (1, 384, 2, 128), (2, 200, 2, 64)])
def test_flash_attention_dropout_matches_reference(B, T, H, d):
    g = torch.Generator(device="cuda").manual_seed(7)
    qkv = (torch.randn(B, T, 3 * H * d, device="cuda", generator=g) * 0.5).half()
    D = H * d
    k, v, q = (qkv[..., i * D:(i + 1) * D].view(B, T, H, d) for i in range(3))
    p_drop, seed = 0.2, 9876543210123
    out, lse = F.flash_attn_fwd(q, k, v, d ** -0.5, True, dropout_p=p_drop, seed=seed)
    F.set_backend("torch")
    try:
        ref, lse_ref = F.flash_attn_fwd(q, k, v, d ** -0.5, True, dropout_p=p_drop, seed=seed)
    finally:
        F.set_backend("auto")
    assert torch.allclose(lse, lse_ref, rtol=1e-3, atol=1e-3)
    assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2), (out.float() - ref.float()).abs().max()
    d_out = torch.randn(B, T, D, device="cuda", generator=g).half()
    grads = {}
    for backend in ("auto", "torch"):
        F.set_backend(backend)
        try:
            dqkv = torch.zeros_like(qkv)
            dk, dv, dq = (dqkv[..., i * D:(i + 1) * D].view(B, T, H, d) for i in range(3))
            F.flash_attn_bwd(q, k, v, out, d_out, lse, d ** -0.5, True, dq, dk, dv, dropout_p=p_drop, seed=seed)
            grads[backend] = dqkv.float()
        finally:
            F.set_backend("auto")
    err = (grads["auto"] - grads["torch"]).abs().max().item()
    assert err <= 3e-2 * grads["torch"].abs().max().item() + 2e-3, err
    # without dropout the same call gives a different (undropped) result
    out0, _ = F.flash_attn_fwd(q, k, v, d ** -0.5, True)
    assert (out0.float() - out.float()).abs().max().item() > 1e-2


def test_wait_on_a_flag_that_nothing_sets_times_out_and_the_context_stays_usable():
    """The bounded wait for a peer's arrival flag: nothing ever publishes the awaited epoch, so after its limit
    (4 s) the kernel gives up, leaves a code in the status word and returns.  While the word is set, kernels
    that check it do no work; once the host has read (and thereby cleared) it, everything runs as before."""
    import time

    lib = _lib.kernels()
    _status_ok()
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    status = _lib.status_word(torch.device("cuda"))
    t0 = time.time()
    rc = lib.msq_comm_wait_flags(_lib.ptr(flags), 0, 4, 0, 0, 1, _lib.ptr(status), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 2.0 < waited < 30.0, waited
    # a GEMM launched while the word is set returns without touching its output
    a = torch.randn(256, 128, device="cuda", dtype=torch.float16)
    w = torch.randn(256, 128, device="cuda", dtype=torch.float16)
    out = torch.full((256, 256), 7.0, device="cuda", dtype=torch.float16)
    F.gemm(a, w, out=out)
    torch.cuda.synchronize()
    assert float(out.float().min()) == 7.0 and float(out.float().max()) == 7.0
    code = _lib.check_status("cuda")
    assert code == 5, code  # ST_TIMEOUT_PEER_FLAG; reading clears the word
    F.gemm(a, w, out=out)
    _close(out, a.float() @ w.float().t(), torch.float16)
    _status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,D,affine", [(64, 2048, True), (37, 768, True), (300, 4096, False), (5, 264, True)])
def test_rms_norm_forward_backward(dtype, rows, D, affine):
    from metaseq_b200.modules.layer_norm import RMSNorm

    torch.manual_seed(rows + D)
    mod = RMSNorm(D, eps=1e-5, elementwise_affine=affine).cuda().to(dtype)
    if affine:
        with torch.no_grad():
            mod.weight.copy_(torch.randn(D, device="cuda").to(dtype))
    x = torch.randn(rows, D, device="cuda", dtype=dtype, requires_grad=True)
    dy = torch.randn(rows, D, device="cuda", dtype=dtype)
    before = _lib.launch_count()
    y = mod(x)
    assert _lib.launch_count() == before + 1
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = mod.weight.detach().float().requires_grad_(True) if affine else None
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5)
    if affine:
        yr = yr * wr
    yr.backward(dy.float())
    _close(y, yr, dtype)
    _close(x.grad, xr.grad, dtype, scale=4.0)
    if affine:
        _close(mod.weight.grad, wr.grad, dtype, scale=float(rows) ** 0.5 * 2)
    _status_ok()


def test_top_p_sampling_kernel_matches_the_sorted_definition():
    torch.manual_seed(21)
    rows, V = 64, 50272
    logits = torch.randn(rows, V, device="cuda") * 3
    logits[:, 1] = float("-inf")  # banned token
    logits[::5, 100:40000] = float("-inf")
    lprobs = torch.log_softmax(logits, -1)
    u = torch.rand(rows, device="cuda")
    # a vanishing nucleus is the arg-max
    lp, tok = F.sample_top_p(lprobs, 1e-7, u)
    assert torch.equal(tok, lprobs.argmax(-1)) and torch.equal(lp, lprobs.max(-1).values)
    # against the same draw written with sort / cumsum (identical uniforms)
    per_row_p = torch.linspace(0.3, 0.95, rows, device="cuda")
    for p in (0.9, 0.5, 1.0, per_row_p):
        before = _lib.launch_count()
        lp, tok = F.sample_top_p(lprobs, p, u)
        assert _lib.launch_count() == before + 1
        F.set_backend("torch")
        try:
            lp_ref, tok_ref = F.sample_top_p(lprobs, p, u)
        finally:
            F.set_backend("auto")
        assert torch.equal(lp, lprobs.gather(-1, tok[:, None]).squeeze(-1))
        assert (tok != 1).all() and torch.isfinite(lp).all()
        # every token lies in the nucleus of the sorted definition (ties with its last member included)
        probs = lprobs.exp()
        sp, _ = probs.sort(descending=True, dim=-1)
        cs = sp.cumsum(-1)
        pp = p.reshape(-1, 1) if torch.is_tensor(p) else p
        last = ((cs - sp) < pp).long().sum(-1, keepdim=True).clamp(min=1) - 1
        thr = sp.gather(-1, last).squeeze(-1)
        chosen_p = probs.gather(-1, tok[:, None]).squeeze(-1)
        assert (chosen_p >= thr * (1 - 1e-4)).all()
        # cumulative sums in a different order move a draw across a token boundary only rarely
        assert (tok == tok_ref).float().mean().item() >= 0.9
    # frequencies over many rows with one distribution
    V2, n = 96, 40000
    base = torch.log_softmax(torch.randn(V2, device="cuda") * 1.5, -1)
    many = base.expand(n, V2).contiguous()
    _, tok = F.sample_top_p(many, 0.8, torch.rand(n, device="cuda"))
    pr = base.exp()
    sp, si = pr.sort(descending=True)
    keep = (sp.cumsum(0) - sp) < 0.8
    expect = torch.zeros(V2, device="cuda")
    expect[si[keep]] = sp[keep] / sp[keep].sum()
    freq = torch.bincount(tok, minlength=V2).float() / n
    assert (freq[expect == 0] == 0).all()
    assert (freq - expect).abs().max().item() < 0.01
    _status_ok()



@pytest.mark.parametrize("pdt,gdt", [(torch.float16, torch.float16), (torch.bfloat16, torch.bfloat16),
                                     (torch.float32, torch.float16), (torch.float32, torch.float32)])
def test_adamw_list_form_matches_one_launch_per_tensor(pdt, gdt):
    torch.manual_seed(4)
    sizes = [8 * 1000, 12345, 7, 262144 + 3, 64]
    kw = dict(lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3)

    def make():
        g = torch.Generator(device="cuda").manual_seed(9)
        items = []
        for i, n in enumerate(sizes):
            base = torch.randn(n + 8, device="cuda", generator=g)
            off = 1 if i == 3 else 0  # one parameter whose storage is not 16-byte aligned
            p = base[off:off + n].to(pdt) if pdt != torch.float32 else base[off:off + n].clone()
            gr = (torch.randn(n, device="cuda", generator=g) * 0.1).to(gdt)
            m = torch.randn(n, device="cuda", generator=g) * 0.01
            v = torch.rand(n, device="cuda", generator=g) * 0.01
            items.append((p.contiguous(), gr, m, v))
        return items

    ctrl = torch.tensor([0.5, 0.0, 0.0, 1.0], device="cuda")
    one, many = make(), make()
    for it in one:
        F.adamw_step(*it, ctrl=ctrl, **kw)
    before = _lib.launch_count()
    F.adamw_step_multi(many, ctrl=ctrl, **kw)
    assert _lib.launch_count() == before + 1
    for a, b in zip(one, many):
        for x, y in zip(a, b):
            torch.testing.assert_close(x.float(), y.float(), rtol=1e-6, atol=1e-7)
    # the skip flag leaves everything untouched
    skip = torch.tensor([1.0, 1.0, 0.0, 1.0], device="cuda")
    snap = [[t.clone() for t in it] for it in many]
    F.adamw_step_multi(many, ctrl=skip, **kw)
    for a, b in zip(snap, many):
        for x, y in zip(a, b):
            assert torch.equal(x, y)
    _status_ok()


def test_adam_with_fp16_statistics_on_the_kernel_path():
    """Moments kept as scaled fp16 between steps: the kernel updates fp32 working copies, and the result follows the
    fp32-moment optimizer to within the quantisation of the moments."""
    from metaseq_b200.optim.adam import Adam

    torch.manual_seed(0)
    shapes = [(1024, 64), (4096,), (333,)]
    full = [torch.nn.Parameter(torch.randn(*s, device="cuda")) for s in shapes]
    half = [torch.nn.Parameter(p.detach().clone()) for p in full]
    a = Adam(full, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    b = Adam(half, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, use_fp16_stats=True)
    gen = torch.Generator(device="cuda").manual_seed(1)
    for _ in range(5):
        for p, q in zip(full, half):
            g = torch.randn(p.shape, device="cuda", generator=gen) * 1e-3
            p.grad, q.grad = g.clone(), g.clone()
        before = _lib.launch_count()
        b.step()
        assert _lib.launch_count() > before  # the update itself is the native kernel
        a.step()
    for p, q in zip(full, half):
        st = b.state[q]
        assert st["exp_avg"].dtype == torch.float16 and st["exp_avg_sq"].dtype == torch.float16
        assert st["exp_avg_scale"].is_cuda  # no host synchronisation for the scale
        assert (p - q).abs().max().item() < 5e-4
    _status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (600, 6288, 256), (1024, 1000, 512)])
def test_gemm_row_statistics_fold_into_the_log_sum_exp(dtype, M, N, K):
    """The logits product's epilogue leaves per-tile (max, sum-exp) of every row over the stored values; folded over
    the tiles they give the row's log-sum-exp, and the cross entropy built on them equals the fp32 oracle."""
    torch.manual_seed(21)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(dtype)
    w = (torch.randn(N, K, device="cuda") * 0.5).to(dtype)
    out, stats = F.gemm_with_row_stats(a, w)
    assert stats is not None and stats[0].shape == (math.ceil(N / 256), M)
    want = _ref(F.gemm, a, w)
    _close(out, want, dtype, scale=4.0)
    m = stats[0].max(dim=0)[0]
    lse = m + torch.log((stats[1] * torch.exp(stats[0] - m)).sum(dim=0))
    torch.testing.assert_close(lse, torch.logsumexp(out.float(), dim=1), rtol=1e-4, atol=1e-3)
    target = torch.randint(0, N, (M,), device="cuda")
    target[::5] = 1
    l1, l2 = out.clone(), out.clone()
    loss = F.cross_entropy_from_row_stats(l1, target, 1, 64.0, stats)
    lossr, _ = _ref(F.cross_entropy_fwd_bwd, l2, target, 1, 64.0, True)
    torch.testing.assert_close(loss, lossr, rtol=1e-3, atol=2e-3)
    _close(l1, l2, dtype, scale=2.0)
    _status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("per_row", [True, False])
def test_scale_rows_relative_to_the_factor_already_applied(dtype, per_row):
    torch.manual_seed(5)
    rows, cols = 200, 512
    x = torch.randn(rows, cols, device="cuda", dtype=dtype)
    keep = x.clone()
    g = torch.full((rows if per_row else 1,), 128.0, device="cuda")
    F.scale_rows_(x, g, ref=128.0)
    assert torch.equal(x, keep)  # the expected factor arrived: nothing is rewritten
    if per_row:
        g[::3] = 0.0
        g[1::3] = 64.0
    else:
        g[0] = 32.0
    F.scale_rows_(x, g, ref=128.0)
    want = keep.float() * (g / 128.0).reshape(-1, 1)
    _close(x, want, dtype)


def test_cross_entropy_applies_the_announced_loss_scale_in_the_forward_pass():
    """With the upstream factor announced, the gradient leaves the forward pass already scaled and the backward pass
    only checks; a different factor in backward is still honoured."""
    from metaseq_b200.ops import autograd as ops_ag

    torch.manual_seed(9)
    rows, V = 512, 4096
    x = (torch.randn(rows, 256, device="cuda") * 0.5).half().requires_grad_(True)
    w = (torch.randn(V, 256, device="cuda") * 0.2).half().requires_grad_(True)
    target = torch.randint(2, V, (rows,), device="cuda")

    def run(hint, upstream):
        ops_ag.set_upstream_grad_hint(hint)
        try:
            x.grad = w.grad = None
            logits = ops_ag.linear(x, w, row_stats=True)
            assert getattr(logits, "_msq_row_stats", None) is not None
            loss = ops_ag.cross_entropy_sum(logits, target, 1)
            (loss * upstream).backward()
            return float(loss), x.grad.clone(), w.grad.clone()
        finally:
            ops_ag.set_upstream_grad_hint(None)

    l0, gx0, gw0 = run(None, 64.0)
    l1, gx1, gw1 = run(64.0, 64.0)
    l2, gx2, gw2 = run(8.0, 64.0)
    assert l0 == pytest.approx(l1, rel=1e-5) and l0 == pytest.approx(l2, rel=1e-5)
    for a, b in ((gx0, gx1), (gw0, gw1), (gx0, gx2), (gw0, gw2)):
        torch.testing.assert_close(a.float(), b.float(), rtol=2e-2, atol=2e-2 * float(a.float().abs().max()))
    ref = torch.nn.functional.cross_entropy(x.detach().float() @ w.detach().float().t(), target, reduction="sum")
    assert l0 == pytest.approx(float(ref), rel=2e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_sum_of_squares_list_form_matches_the_per_tensor_kernel(dtype):
    from metaseq_b200 import utils

    torch.manual_seed(13)
    sizes = [1, 7, 4096, 100_003, 2_000_000, 8, 33]
    big = torch.randn(sum(sizes) + 64, device="cuda").to(dtype)
    tensors, off = [], 3  # odd offsets: some tensors are not 16-byte aligned
    for n in sizes:
        tensors.append(big[off:off + n])
        off += n + 1
    out = torch.full((1,), 5.0, device="cuda")
    before = _lib.launch_count()
    F.sumsq_multi(tensors, out, True)
    assert _lib.launch_count() == before + 1
    want = 5.0 + sum(float(t.double().pow(2).sum()) for t in tensors)
    assert float(out) == pytest.approx(want, rel=2e-5)
    again = torch.zeros(1, device="cuda")
    F.sumsq_multi(tensors, again, False)
    twice = torch.zeros(1, device="cuda")
    F.sumsq_multi(tensors, twice, False)
    assert float(again) == float(twice)  # same bits from call to call
    norm = utils.multi_tensor_l2_norm(tensors)
    assert float(norm) == pytest.approx(math.sqrt(want - 5.0), rel=2e-5)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_inf_norm_and_scale_list_forms(dtype):
    from metaseq_b200 import utils

    torch.manual_seed(14)
    sizes = [5, 4096, 70_001, 1_000_000, 9]
    big = torch.randn(sum(sizes) + 64, device="cuda").to(dtype)
    tensors, off = [], 1
    for n in sizes:
        tensors.append(big[off:off + n])
        off += n + 1
    out = torch.zeros(1, device="cuda")
    before = _lib.launch_count()
    F.absmax_multi(tensors, out)
    assert _lib.launch_count() == before + 1
    assert float(out) == max(float(t.float().abs().max()) for t in tensors)
    copies = [t.clone() for t in tensors]
    coef = torch.tensor([0.25], device="cuda")
    before = _lib.launch_count()
    F.scale_multi_(copies, coef, host_scale=2.0)
    assert _lib.launch_count() == before + 1
    for c, t in zip(copies, tensors):
        assert torch.equal(c, (t.float() * 0.5).to(dtype))
    # clipping a parameter list: inf-norm and l2-norm through the list kernels equal the PyTorch statement
    params = [torch.nn.Parameter(torch.zeros_like(t)) for t in tensors]
    for norm_type in ("l2", "inf"):
        for p_, t in zip(params, tensors):
            p_.grad = t.clone()
        total = utils.clip_grad_norm_(params, 1.0, norm_type=norm_type)
        flat = torch.cat([t.float().reshape(-1) for t in tensors])
        want = flat.abs().max() if norm_type == "inf" else flat.norm()
        assert float(total) == pytest.approx(float(want), rel=2e-5)
        c = min(1.0, 1.0 / (float(want) + 1e-6))
        for p_, t in zip(params, tensors):
            tol = 1e-6 if dtype == torch.float32 else (1e-3 if dtype == torch.float16 else 8e-3)
            assert torch.allclose(p_.grad.float(), t.float() * c, rtol=tol, atol=tol * 1e-2)
    bad = [t.clone() for t in tensors]
    bad[2][17] = float("nan")
    assert float(F.absmax_multi(bad, out)) == float("inf")


def test_bias_gradient_single_launch_leaves_its_scratch_clean():
    torch.manual_seed(15)
    for rows, N in [(3001, 776), (16384, 2048), (70, 8192), (3001, 776)]:
        x = torch.randn(rows, N, device="cuda").to(torch.bfloat16)
        dst = torch.randn(N, device="cuda").to(torch.bfloat16)
        keep = dst.clone()
        before = _lib.launch_count()
        F.colsum(x, out16=dst, accumulate=True)
        assert _lib.launch_count() == before + 1
        want = keep.float() + x.float().sum(0)
        assert (dst.float() - want).abs().max() <= 0.02 * want.abs().max() + 0.05
        F.colsum(x, out16=dst, accumulate=False)  # the second call starts from a scratch the first left at zero
        want = x.float().sum(0)
        assert (dst.float() - want).abs().max() <= 0.01 * want.abs().max() + 0.05


def _attn_fwd_bwd(q, k, v, qkv, d_out, scale, use_ref, **masks):
    """Forward and backward through the kernels (or the PyTorch restatement): returns (out, lse, dqkv)."""
    B, T, H, d = q.shape
    D = H * d
    fwd = (lambda *a, **kw: _ref(F.flash_attn_fwd, *a, **kw)) if use_ref else F.flash_attn_fwd
    bwd = (lambda *a, **kw: _ref(F.flash_attn_bwd, *a, **kw)) if use_ref else F.flash_attn_bwd
    out, lse = fwd(q, k, v, scale, True, **masks)
    dqkv = torch.zeros_like(qkv)
    dk, dv, dq = (dqkv[..., i * D:(i + 1) * D].view(B, T, H, d) for i in range(3))
    bwd(q, k, v, out, d_out, lse, scale, True, dq, dk, dv, **masks)
    return out, lse, dqkv


def _document_starts(B, T, mean_len, seed):
    g = torch.Generator().manual_seed(seed)
    starts = torch.zeros(B, T, dtype=torch.int32)
    for b in range(B):
        t = 0
        while t < T:
            n = int(torch.randint(1, 2 * mean_len, (1,), generator=g))
            starts[b, t:t + n] = t
            t += n
    return starts.cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [80, 96, 32])
@pytest.mark.parametrize("T", [256, 200])
def test_flash_attention_head_sizes_between_the_native_ones(dtype, d, T):
    """Head sizes 80 and 96 (OPT-2.7B, OPT-760M) run the 128-wide kernels on zero-filled columns, 32 the 64-wide."""
    torch.manual_seed(31)
    B, H = 2, 3
    qkv, q, k, v = _attn_inputs(B, T, H, d, dtype)
    d_out = (torch.randn(B, T, H * d, device="cuda") * 0.5).to(dtype)
    before = _lib.launch_count()
    got = _attn_fwd_bwd(q, k, v, qkv, d_out, d ** -0.5, False)
    assert _lib.launch_count() > before  # the kernel path, not the PyTorch restatement
    want = _attn_fwd_bwd(q, k, v, qkv, d_out, d ** -0.5, True)
    _status_ok()
    _close(got[0], want[0], dtype)
    torch.testing.assert_close(got[1], want[1], rtol=2e-3, atol=2e-3)
    _close(got[2], want[2], dtype, scale=4.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,T,mean_len", [(64, 512, 40), (128, 384, 150), (64, 1000, 300), (96, 256, 20)])
def test_flash_attention_document_starts(dtype, d, T, mean_len):
    """Queries see only the keys of their own document; kv blocks before a tile's documents are skipped."""
    torch.manual_seed(32)
    B, H = 2, 2
    qkv, q, k, v = _attn_inputs(B, T, H, d, dtype)
    d_out = (torch.randn(B, T, H * d, device="cuda") * 0.5).to(dtype)
    starts = _document_starts(B, T, mean_len, 5)
    got = _attn_fwd_bwd(q, k, v, qkv, d_out, d ** -0.5, False, doc_start=starts)
    want = _attn_fwd_bwd(q, k, v, qkv, d_out, d ** -0.5, True, doc_start=starts)
    plain = _attn_fwd_bwd(q, k, v, qkv, d_out, d ** -0.5, True)
    _status_ok()
    _close(got[0], want[0], dtype)
    torch.testing.assert_close(got[1], want[1], rtol=2e-3, atol=2e-3)
    _close(got[2], want[2], dtype, scale=4.0)
    assert (want[0].float() - plain[0].float()).abs().max() > 1e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,T", [(64, 384), (128, 200)])
def test_flash_attention_alibi(dtype, d, T):
    from metaseq_b200.modules.attention_bias import alibi_slopes

    torch.manual_seed(33)
    B, H = 2, 4
    qkv, q, k, v = _attn_inputs(B, T, H, d, dtype)
    d_out = (torch.randn(B, T, H * d, device="cuda") * 0.5).to(dtype)
    slopes = torch.tensor(alibi_slopes(H), device="cuda")
    starts = _document_starts(B, T, 90, 6)
    for masks in (dict(alibi_slopes=slopes), dict(alibi_slopes=slopes, doc_start=starts)):
        got = _attn_fwd_bwd(q, k, v, qkv, d_out, d ** -0.5, False, **masks)
        want = _attn_fwd_bwd(q, k, v, qkv, d_out, d ** -0.5, True, **masks)
        _status_ok()
        _close(got[0], want[0], dtype)
        torch.testing.assert_close(got[1], want[1], rtol=2e-3, atol=2e-3)
        _close(got[2], want[2], dtype, scale=4.0)


def test_flash_attention_at_the_benchmarked_shape():
    """T = 2048 with B * H = 256 (the OPT-1.3B training shape): enough CTAs to fill every SM several times.  The
    oracle runs per slice of heads to bound its [B, H, T, T] scores."""
    torch.manual_seed(34)
    B, T, H, d = 8, 2048, 32, 64
    qkv, q, k, v = _attn_inputs(B, T, H, d, torch.float16)
    D = H * d
    d_out = (torch.randn(B, T, D, device="cuda") * 0.5).half()
    out, lse, dqkv = _attn_fwd_bwd(q, k, v, qkv, d_out, d ** -0.5, False)
    _status_ok()
    for b, h0 in ((0, 0), (3, 8), (7, 28)):
        sl = slice(h0, h0 + 4)
        qs, ks, vs = (t[b:b + 1, :, sl].contiguous() for t in (q, k, v))
        sub = torch.cat([ks.reshape(1, T, -1), vs.reshape(1, T, -1), qs.reshape(1, T, -1)], dim=-1)
        kk, vv, qq = (sub[..., i * 4 * d:(i + 1) * 4 * d].view(1, T, 4, d) for i in range(3))
        do = d_out[b:b + 1].view(1, T, H, d)[:, :, sl].reshape(1, T, 4 * d).contiguous()
        o_r, lse_r, dsub = _attn_fwd_bwd(qq, kk, vv, sub, do, d ** -0.5, True)
        _close(out[b:b + 1].view(1, T, H, d)[:, :, sl].reshape(1, T, 4 * d), o_r, torch.float16)
        torch.testing.assert_close(lse[b:b + 1, sl], lse_r, rtol=2e-3, atol=2e-3)
        got = torch.cat([dqkv[b:b + 1, :, i * D:(i + 1) * D].view(1, T, H, d)[:, :, sl].reshape(1, T, 4 * d)
                         for i in range(3)], dim=-1)
        _close(got, dsub, torch.float16, scale=4.0)
