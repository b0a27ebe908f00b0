"""Error paths that must leave the context usable: a device-side bounded wait that runs out, and first
uses that a recording must not swallow.  No GPU fault is provoked anywhere: the wait test withholds one
asynchronous copy, so a barrier is simply never completed and the kernel's own poll limit ends the wait."""
import numpy as np
import pytest

from oracle.wasm_oracle import T, WasmOracle

pytestmark = pytest.mark.gpu


def _product(ctx, rng, M=256, K=512, N=256):
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
    return a, w, ctx.upload(a, M, K), ctx.uploadF16(w, K, N)


def test_bounded_wait_runs_out_and_context_survives(pkg):
    """One thread block of a tensor-core product never gets K chunk 3 of its first tile: the MMA warp's wait on
    that stage gives up after `wait_limit` polls (a few milliseconds here, not the default second), the kernel
    records a status word, unwinds, frees its TMEM and returns; fa_sync reports FA_ERR_TIMEOUT; the next product
    on the same context is correct."""
    ctx = pkg.CudaContext(0)
    try:
        rng = np.random.default_rng(3)
        a, w, A, Wt = _product(ctx, rng)
        ref = WasmOracle(threads=True).matmul(T(a, 256, 512), T(w, 512, 256)).array()
        good = ctx.download(ctx.matmul(A, Wt)).reshape(256, 256)  # also builds the packed weight copy
        assert np.abs(good - ref).max() <= 2e-2
        ctx.setOption("wait_limit", 20000)
        ctx.setOption("tc_test_withhold_chunk", 3)
        ctx.matmul(A, Wt)
        with pytest.raises(pkg.CudaError) as ei:
            ctx.sync()
        assert ei.value.code == 5 and "bounded wait ran out" in str(ei.value)  # FA_ERR_TIMEOUT
        ctx.setOption("wait_limit", 1 << 24)
        again = ctx.download(ctx.matmul(A, Wt)).reshape(256, 256)
        assert np.array_equal(again, good)
        ctx.sync()  # status word was cleared: no stale error
    finally:
        ctx.destroy()


def test_bounded_wait_runs_out_in_the_pair_kernel(pkg):
    """The same for a product large enough to run on pairs of thread blocks (two CTAs of a cluster sharing one MMA):
    the leader of pair 0 never announces K chunk 2 of its first tile, every role of both CTAs gives up on its own
    bounded wait, both leave through the cluster barrier, and the context keeps working."""
    ctx = pkg.CudaContext(0)
    try:
        rng = np.random.default_rng(6)
        M, K, N = 6016, 256, 1024
        a = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
        A, Wt = ctx.upload(a, M, K), ctx.uploadF16(w, K, N)
        good = ctx.download(ctx.matmul(A, Wt)).reshape(M, N)
        rows = np.arange(0, M, 97)
        ref = WasmOracle(threads=True).matmul(T(a[rows], len(rows), K), T(w, K, N)).array()
        assert np.abs(good[rows] - ref).max() <= 2e-2
        ctx.setOption("wait_limit", 20000)
        ctx.setOption("tc_test_withhold_chunk", 2)
        ctx.matmul(A, Wt)
        with pytest.raises(pkg.CudaError) as ei:
            ctx.sync()
        assert ei.value.code == 5 and "bounded wait ran out" in str(ei.value)  # FA_ERR_TIMEOUT
        ctx.setOption("wait_limit", 1 << 24)
        again = ctx.download(ctx.matmul(A, Wt)).reshape(M, N)
        assert np.array_equal(again, good)
        ctx.sync()
    finally:
        ctx.destroy()


def test_bounded_wait_runs_out_in_the_prediction_network_kernel(pkg):
    """The TDT decoder's exact-f32 products stream their operands through per-warp rings of bulk copies: warp 0 of
    block 0 never issues stage 2 of the first LSTM layer's first evaluation, its bounded wait runs out, the decode
    returns FA_ERR_TIMEOUT and the next decode on the same context gives the reference's tokens."""
    from fluidaudio_web_b200.engines import tdt_decoder as td
    from oracle.tdt_oracle import TdtOracle

    ctx = pkg.CudaContext(0)
    try:
        W, Tn = 4, 24
        w = td.synth_tdt_weights(5)
        proj = np.random.default_rng(424).standard_normal((W, Tn, 640)).astype(np.float32)
        want = TdtOracle(w, int8=True, threads=4).decode_proj_batch(proj, W, Tn)
        dec = td.TdtDecoder(ctx, w, int8=True)
        P = ctx.upload(proj.reshape(W * Tn, 640), W * Tn, 640)
        ctx.setOption("wait_limit", 20000)
        ctx.setOption("tc_test_withhold_chunk", 2)
        with pytest.raises(pkg.CudaError) as ei:
            dec.decode_proj(P, W, Tn)
        assert ei.value.code == 5 and "bounded wait ran out" in str(ei.value)  # FA_ERR_TIMEOUT
        ctx.setOption("wait_limit", 1 << 24)
        got = dec.decode_proj(P, W, Tn)
        for wi in range(W):
            assert got[wi][0].tolist() == want[wi][0].tolist() and got[wi][1].tolist() == want[wi][1].tolist()
        dec.free()
    finally:
        ctx.destroy()


def test_first_use_of_a_weight_inside_a_recording_is_refused(pkg):
    """The packed tensor-core copy of a weight is built on first use.  Inside a recording that step would only be
    captured while the handle already looked ready, and an eager product before the first replay would read
    unwritten memory; the library refuses instead, and after one eager run recording works and eager use between
    recording and replay is correct."""
    ctx = pkg.CudaContext(0)
    try:
        rng = np.random.default_rng(4)
        a, w, A, Wt = _product(ctx, rng)
        ref = WasmOracle(threads=True).matmul(T(a, 256, 512), T(w, 512, 256)).array()
        with pytest.raises(pkg.CudaError, match="eagerly before"):
            ctx.recordBatch(lambda: ctx.matmul(A, Wt))
        ctx.freeTensor(ctx.matmul(A, Wt))  # once eagerly
        batch, out = ctx.recordBatch(lambda: ctx.matmul(A, Wt))
        eager = ctx.download(ctx.matmul(A, Wt)).reshape(256, 256)  # before any replay
        assert np.abs(eager - ref).max() <= 2e-2
        batch.launch()
        assert np.array_equal(ctx.download(out).reshape(256, 256), eager)
        batch.free()
    finally:
        ctx.destroy()


def test_row_operand_from_before_a_recording_is_repacked_per_replay(pkg):
    """A row operand uploaded before the recording and first used inside it carries no packed copy: it is packed
    into per-call scratch on every replay, so a replay sees new contents written into it in between."""
    ctx = pkg.CudaContext(0)
    try:
        rng = np.random.default_rng(5)
        a, w, A, Wt = _product(ctx, rng)
        A2 = ctx.upload(a, 256, 512)  # never used eagerly as an operand
        ctx.freeTensor(ctx.matmul(A, Wt))
        batch, out = ctx.recordBatch(lambda: ctx.matmul(A2, Wt))
        want = ctx.download(ctx.matmul(A2, Wt)).reshape(256, 256)  # eager, before the first replay
        batch.launch()
        assert np.array_equal(ctx.download(out).reshape(256, 256), want)
        batch.free()
    finally:
        ctx.destroy()


def test_mark_and_wait_mark_between_contexts(pkg):
    """Ordering between two contexts of one GPU: waiting for a context that never marked is a no-op, a marked point
    can be waited for, and neither call is accepted while a recording is open (it would not be part of it)."""
    a, b = pkg.CudaContext(0), pkg.CudaContext(0)
    try:
        rng = np.random.default_rng(9)
        x, w, X, Wt = _product(a, rng)
        b.waitMark(a)  # nothing marked yet
        y = a.matmul(X, Wt)
        a.mark()
        b.waitMark(a)
        x2, w2, X2, Wt2 = _product(b, rng)
        y2 = b.matmul(X2, Wt2)
        assert np.abs(b.download(y2).reshape(x2.shape[0], -1) - x2 @ w2).max() <= 2e-2
        assert np.abs(a.download(y).reshape(x.shape[0], -1) - x @ w).max() <= 2e-2

        def body():
            with pytest.raises(pkg.CudaError):
                a.mark()
            with pytest.raises(pkg.CudaError):
                a.waitMark(b)
            return a.matmul(X, Wt)

        batch, _ = a.recordBatch(body)
        batch.launch()
        a.sync()
        batch.free()
    finally:
        a.destroy()
        b.destroy()
