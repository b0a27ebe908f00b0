"""The allocation-free int8 product (fa_matmul_int8_static) against the regular entry point.

Collected last on purpose: a failure here cannot hide the results of the other GPU tests in a run
that stops at the first failure.  The entry point serves hosts that may not allocate device memory
at call time, so its scratch is a fixed array inside the library that every call shares; two calls
in a row with different shapes check that nothing left over from the first call leaks into the second.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_pair(ctx, rng, M, K, N, act, check_alloc=True):
    a = rng.standard_normal((M, K)).astype(np.float32)
    wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    sc = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    A, S, B = ctx.upload(a, M, K), ctx.upload(sc, 1, N), ctx.upload(bias, 1, N)
    ref = ctx.download(ctx.matmulInt8(A, ctx.uploadBytes(wq), S, N, K, bias=B, act=act)).reshape(M, N)
    # the raw int8 bytes ride in an f32 tensor (uploads are plain byte copies), which gives a device pointer
    W = ctx.upload(wq.reshape(-1).view(np.float32), 1, K * N // 4)
    Y = ctx.alloc(M, N)
    ptrs = [ctx.devicePtr(t) for t in (A, W, S, B, Y)]
    ctx.sync()
    # the property the entry point exists for: the call itself makes no device allocation - none through the
    # library's pool (counters unchanged, not even a pool hit) and none behind its back (free memory unchanged)
    before, free_before = ctx.memStats(), _free_bytes()
    ctx.matmulInt8Static(ptrs[0], ptrs[1], ptrs[2], ptrs[3], act, ptrs[4], M, N, K)
    after, free_after = ctx.memStats(), _free_bytes()
    if check_alloc:
        for key in ("created", "createdBytes", "reused", "poolBytes"):
            assert after[key] == before[key], (key, before, after)
        assert free_after == free_before
    got = ctx.download(Y).reshape(M, N)
    return got, ref


def _free_bytes():
    import torch

    return torch.cuda.mem_get_info(0)[0]


def test_static_scratch_entry_matches_regular_entry_twice(ctx):
    rng = np.random.default_rng(7)
    # the first call on a device resolves the scratch array's address (documented set-up step)
    _run_pair(ctx, rng, 128, 256, 256, "none", check_alloc=False)
    got1, ref1 = _run_pair(ctx, rng, 512, 1024, 4096, "none")
    got2, ref2 = _run_pair(ctx, rng, 200, 328, 136, "relu")  # smaller, ragged: stale bytes would show here
    # same kernels and same arithmetic as the regular entry point: identical results
    assert np.array_equal(got1, ref1)
    assert np.array_equal(got2, ref2)


def test_static_scratch_entry_rejects_oversize(ctx, pkg):
    a = ctx.alloc(1, 64)
    with pytest.raises(pkg.CudaError, match="outside"):
        ctx.matmulInt8Static(ctx.devicePtr(a), ctx.devicePtr(a), ctx.devicePtr(a), None, "none", ctx.devicePtr(a), 513, 128, 64)
    with pytest.raises(pkg.CudaError, match="outside"):
        ctx.matmulInt8Static(ctx.devicePtr(a), ctx.devicePtr(a), ctx.devicePtr(a), None, "none", ctx.devicePtr(a), 16, 128, 4096)
    with pytest.raises(pkg.CudaError, match="static scratch holds"):
        ctx.matmulInt8Static(ctx.devicePtr(a), ctx.devicePtr(a), ctx.devicePtr(a), None, "none", ctx.devicePtr(a), 16, 8192, 2048)
