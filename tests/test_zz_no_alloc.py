"""The allocation-free sum-of-squares entry point, called through its exported C symbol.

Some users of the kernel library cannot ask for device memory: helper threads (checkpoint
writer, watchdog) that run beside a training step whose caching allocator already owns the
GPU, and C/C++ programs that link the library without PyTorch.  For them
``msq_sumsq_noalloc`` keeps its partial sums in an array inside the library.  This test calls
it twice in a row on different inputs and checks both results against ``msq_sumsq``, the
ordinary entry point that takes a caller-allocated scratch buffer.  It lives in a file that
pytest collects last so that a failure here cannot hide the outcome of any other test.
"""
import ctypes

import pytest
import torch

from metaseq_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _symbols():
    lib = ctypes.CDLL(str(_lib.kernels_path()))
    P, L, I = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    new = lib.msq_sumsq_noalloc
    new.argtypes = [P, L, I, P, I, P]
    new.restype = I
    old = lib.msq_sumsq
    old.argtypes = [P, L, I, P, P, I, P]
    old.restype = I
    parts = lib.msq_sumsq_parts
    parts.argtypes = [L]
    parts.restype = I
    return new, old, parts


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_no_alloc_sumsq_matches_regular_entry_point(dtype):
    new, old, parts = _symbols()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = _lib.dtype_code(dtype)
    torch.manual_seed(11)
    # the second call is shorter than the first: slots left over from call one must not leak in
    for n in (3_000_017, 4099):
        g = (torch.randn(n, device="cuda") * 2).to(dtype)
        want = torch.zeros(1, dtype=torch.float32, device="cuda")
        scratch = torch.empty(parts(n), dtype=torch.float32, device="cuda")
        assert old(g.data_ptr(), n, code, scratch.data_ptr(), want.data_ptr(), 0, stream) == 0
        got = torch.full((1,), 123.0, dtype=torch.float32, device="cuda")
        assert new(g.data_ptr(), n, code, got.data_ptr(), 0, stream) == 0
        torch.cuda.synchronize()
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-3)
        ref = g.float().pow(2).sum()
        torch.testing.assert_close(got[0], ref, rtol=1e-4, atol=1e-2)
        # accumulate mode adds to what is already there
        assert new(g.data_ptr(), n, code, got.data_ptr(), 1, stream) == 0
        torch.cuda.synchronize()
        torch.testing.assert_close(got, 2 * want, rtol=1e-5, atol=2e-3)


def test_no_alloc_sumsq_rejects_oversize_and_bad_dtype():
    new, _, _ = _symbols()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.zeros(16, device="cuda")
    out = torch.zeros(1, device="cuda")
    assert new(g.data_ptr(), (1 << 31) + 1, 2, out.data_ptr(), 0, stream) == -20
    assert new(g.data_ptr(), -1, 2, out.data_ptr(), 0, stream) == -20
    assert new(g.data_ptr(), 16, 7, out.data_ptr(), 0, stream) == -21
    torch.cuda.synchronize()
    assert float(out) == 0.0
