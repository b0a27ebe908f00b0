"""Context semantics on the GPU: arenas, pool reuse, staged single-use reads, views, batching,
recorded batches, profiler.  Contract sources: src/gpu/buffer-pool.js:49-135,
src/gpu/compute.js:1101-1136, src/gpu/scheduler.js:17-60,139-180, src/gpu/compute.d.ts:39-45."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_staged_read_is_single_use_and_ordered_at_stage_time(ctx, pkg):
    a = np.arange(12, dtype=np.float32)
    t = ctx.upload(a, 3, 4)
    s = ctx.stageDownload(t)
    ctx.copyRows(t, ctx.upload(np.full(4, 9, np.float32), 1, 4), 0)  # later op must not change the snapshot
    assert np.array_equal(s.read(), a)
    with pytest.raises(pkg.CudaError, match="already consumed"):
        s.read()


def test_nested_batch_throws(ctx, pkg):
    ctx.beginBatch()
    with pytest.raises(pkg.CudaError, match="not re-entrant"):
        ctx.beginBatch()
    ctx.endBatch()
    assert ctx.withBatchSync(lambda: 5) == 5


def test_arena_returns_blocks_to_pool_and_pin_survives(ctx):
    h = ctx.pushArena()
    a = ctx.alloc(64, 64)
    keep = ctx.pin(ctx.alloc(8, 8))
    before = ctx.memStats()
    ctx.popArena(h)
    assert ctx.poolInfo()["bytes"] > 0
    b = ctx.alloc(64, 64)  # exact-size block comes back from the pool
    assert ctx.memStats()["reused"] == before["reused"] + 1
    assert ctx.download(keep).size == 64
    ctx.freeTensor(b)
    ctx.freeTensor(keep)


def test_pin_to_parent_and_out_of_order_close(ctx, pkg):
    outer = ctx.pushArena()
    inner = ctx.pushArena()
    x = ctx.upload(np.ones(4, np.float32), 1, 4)
    y = ctx.pin(ctx.add(x, x), True)  # promoted to the outer arena
    ctx.popArena(inner)
    assert np.array_equal(ctx.download(y), np.full(4, 2, np.float32))
    third = ctx.pushArena()
    ctx.popArena(outer)  # scopes may close out of order
    with pytest.raises(pkg.CudaError):
        ctx.download(y)  # released with the outer arena
    ctx.popArena(third)
    ctx.freeTensor(x)


def test_rows_view_aliases_storage(ctx):
    cache = ctx.alloc(6, 4)
    ctx.copyRows(cache, ctx.upload(np.arange(8, dtype=np.float32), 2, 4), 0)
    v = ctx.rowsView(cache, 2)
    assert (v.rows, v.cols, v.view) == (2, 4, True)
    assert np.array_equal(ctx.download(v), np.arange(8, dtype=np.float32))
    ctx.copyRows(cache, ctx.upload(np.full(4, 7, np.float32), 1, 4), 1)
    assert np.array_equal(ctx.download(v)[4:], np.full(4, 7, np.float32))


def test_bad_shapes_and_handles_fail_loudly(ctx, pkg):
    a, b = ctx.alloc(3, 4), ctx.alloc(5, 6)
    with pytest.raises(pkg.CudaError, match="matmul: A is"):
        ctx.matmul(a, b)
    with pytest.raises(pkg.CudaError, match="block size"):
        ctx.matmulNBits(ctx.alloc(1, 64), ctx.uploadBytes(np.zeros(64, np.uint8)), ctx.alloc(1, 2),
                        ctx.uploadBytes(np.zeros(4, np.uint8)), 2, 64)
    ctx.freeTensor(a)
    with pytest.raises(pkg.CudaError):
        ctx.download(a.__class__(b.h + 8, 1, 1))


def test_pool_cap_reports_out_of_memory(ctx, pkg):
    ctx = pkg.CudaContext(ctx.device)  # a context of its own: the cap is set against a pool nothing else has filled
    try:
        ctx.alloc(64, 64)
        ctx.trimPool(0)
        ctx.setOption("pool_cap_bytes", ctx.memStats()["createdBytes"])  # already above any headroom
        with pytest.raises(pkg.CudaError) as ei:
            ctx.alloc(4096, 4096)
        assert ei.value.code == 3
    finally:
        ctx.destroy()


def test_recorded_batch_replays_with_new_inputs(ctx):
    rng = np.random.default_rng(3)
    M, K, N = 64, 512, 256
    wq = ctx.uploadBytes(rng.integers(-127, 128, (K, N), dtype=np.int8))
    sc = ctx.upload(rng.uniform(1e-3, 1e-2, N).astype(np.float32), 1, N)
    g, b = ctx.upload(np.ones(N, np.float32), 1, N), ctx.upload(np.zeros(N, np.float32), 1, N)
    host = ctx.pinnedArray(M * K)

    def step():
        x = ctx.upload(host, M, K)  # replays re-read the page-locked buffer
        return ctx.layernorm(ctx.matmulInt8(x, wq, sc, N, K, act="relu"), g, b)

    host[:] = rng.standard_normal(M * K).astype(np.float32)
    eager1 = ctx.download(step())
    batch, out = ctx.recordBatch(step)
    batch.launch()
    assert np.array_equal(ctx.download(out), eager1)
    host[:] = rng.standard_normal(M * K).astype(np.float32)
    eager2 = ctx.download(step())
    batch.launch()
    assert np.array_equal(ctx.download(out), eager2)
    assert not np.array_equal(eager1, eager2)
    batch.free()


def test_profiler_reports_labels_and_counts(ctx):
    a = ctx.upload(np.ones(64 * 64, np.float32), 64, 64)
    ctx.startProfile()
    ctx.add(a, a)
    ctx.add(a, a)
    ctx.transpose(a)
    prof = {e["label"]: e for e in ctx.endProfile()}
    assert prof["ewise"]["count"] == 2 and prof["transpose"]["count"] == 1
    assert all(e["ms"] >= 0 for e in prof.values())


def test_recorded_hidden_layer_result_is_fresh_after_every_replay(ctx):
    """A product with a fused activation recorded in a batch writes only its packed f16 form on replay; reading
    its f32 values after each replay must see that replay's result, not the first one's."""
    rng = np.random.default_rng(5)
    M, K, N = 300, 256, 512
    w = (rng.standard_normal((K, N)) / 16).astype(np.float16).astype(np.float32)
    W = ctx.uploadF16(w, K, N)
    host = ctx.pinnedArray(M * K)
    a0 = rng.standard_normal((M, K)).astype(np.float32)
    host[:] = a0.reshape(-1)

    def body():
        return ctx.matmul(ctx.upload(host, M, K), W, dict(act="relu"))

    ctx.freeTensor(body())
    batch, out = ctx.recordBatch(body)
    for scale in (1.0, -2.0, 0.5):
        host[:] = (a0 * scale).reshape(-1)
        batch.launch()
        got = ctx.download(out).reshape(M, N)
        ref = np.maximum((a0 * scale).astype(np.float16).astype(np.float32) @ w, 0)
        assert np.abs(got - ref).max() <= 2e-2 * max(1.0, float(np.abs(ref).max())), scale
    batch.free()
