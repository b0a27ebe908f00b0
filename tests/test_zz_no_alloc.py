"""The allocation-free int8 product (fa_matmul_int8_static) against the regular entry point.

Collected last on purpose: a failure here cannot hide the results of the other GPU tests in a run
that stops at the first failure.  The entry point serves hosts that may not allocate device memory
at call time, so its scratch is a fixed array inside the library that every call shares; two calls
in a row with different shapes check that nothing left over from the first call leaks into the second.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_pair(ctx, rng, M, K, N, act):
    a = rng.standard_normal((M, K)).astype(np.float32)
    wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    sc = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    A, S, B = ctx.upload(a, M, K), ctx.upload(sc, 1, N), ctx.upload(bias, 1, N)
    ref = ctx.download(ctx.matmulInt8(A, ctx.uploadBytes(wq), S, N, K, bias=B, act=act)).reshape(M, N)
    # the raw int8 bytes ride in an f32 tensor (uploads are plain byte copies), which gives a device pointer
    W = ctx.upload(wq.reshape(-1).view(np.float32), 1, K * N // 4)
    Y = ctx.alloc(M, N)
    ctx.matmulInt8Static(ctx.devicePtr(A), ctx.devicePtr(W), ctx.devicePtr(S), ctx.devicePtr(B), act, ctx.devicePtr(Y), M, N, K)
    got = ctx.download(Y).reshape(M, N)
    return got, ref


def test_static_scratch_entry_matches_regular_entry_twice(ctx):
    rng = np.random.default_rng(7)
    stats0 = ctx.memStats()
    got1, ref1 = _run_pair(ctx, rng, 512, 1024, 4096, "none")
    got2, ref2 = _run_pair(ctx, rng, 200, 328, 136, "relu")  # smaller, ragged: stale bytes would show here
    # same kernels and same arithmetic as the regular entry point: identical results
    assert np.array_equal(got1, ref1)
    assert np.array_equal(got2, ref2)
    assert ctx.memStats()["created"] >= stats0["created"]


def test_static_scratch_entry_rejects_oversize(ctx, pkg):
    a = ctx.alloc(1, 64)
    with pytest.raises(pkg.CudaError, match="outside"):
        ctx.matmulInt8Static(ctx.devicePtr(a), ctx.devicePtr(a), ctx.devicePtr(a), None, "none", ctx.devicePtr(a), 513, 128, 64)
    with pytest.raises(pkg.CudaError, match="outside"):
        ctx.matmulInt8Static(ctx.devicePtr(a), ctx.devicePtr(a), ctx.devicePtr(a), None, "none", ctx.devicePtr(a), 16, 128, 4096)
    with pytest.raises(pkg.CudaError, match="static scratch holds"):
        ctx.matmulInt8Static(ctx.devicePtr(a), ctx.devicePtr(a), ctx.devicePtr(a), None, "none", ctx.devicePtr(a), 16, 8192, 2048)
