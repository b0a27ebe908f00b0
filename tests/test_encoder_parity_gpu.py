"""FastConformer encoder forward on the CUDA backend against the same forward on the CPU oracle
(the reference gate for this is scripts/backend-parity.mjs:57-67, WebGPU vs WASM maxΔ < 2e-3 on real
weights).  Random-init stacks amplify rounding differences layer over layer (docs/ORT_REMOVAL.md:121-128),
so the full-size check is teacher-forced per layer: every layer starts from the oracle's input."""
import numpy as np
import pytest

from oracle.wasm_oracle import T, WasmOracle

pytestmark = pytest.mark.gpu


def _eng():
    from fluidaudio_web_b200.engines import fastconformer, synth

    return fastconformer, synth


def test_tiny_encoder_end_to_end(ctx, pkg):
    fc, synth = _eng()
    w = synth.encoder_weights(synth.TINY, seed=3)
    mels = [synth.log_mel(a, 32).reshape(-1) for a in synth.synth_audio(3, samples=16000 * 2, seed=3)]
    ora = WasmOracle(threads=True)
    ref, Tsub = fc.encode_batch(ora, fc.load_encoder(ora, w), mels)
    h = ctx.pushArena()
    got, Tsub2 = fc.encode_batch(ctx, fc.load_encoder(ctx, w), mels)
    out = ctx.download(got).reshape(ref.rows, ref.cols)
    ctx.popArena(h)
    # the reference's exact op sequence (per-window conv loop) gives the same frames as the one-launch form
    h = ctx.pushArena()
    got_ref_seq, _ = fc.encode_batch(ctx, fc.load_encoder(ctx, w), mels, use_fast=False)
    assert np.abs(ctx.download(got_ref_seq).reshape(ref.rows, ref.cols) - out).max() <= 1e-4
    ctx.popArena(h)
    assert Tsub == Tsub2 and (got.rows, got.cols) == (ref.rows, ref.cols)
    # two layers, f16 weights on the device vs f32 on the oracle; outputs are LayerNorm'ed (unit scale)
    assert np.abs(out - ref.array()).max() <= 2e-2


def test_full_width_layer_teacher_forced(ctx, pkg):
    """One real-size conformer block (D=1024, DFF=4096, 8 heads of 128) on 2 windows of 188 frames."""
    fc, synth = _eng()
    cfg = dict(synth.PARAKEET_06B, layers=1)
    w = synth.encoder_weights(cfg, seed=3)
    rng = np.random.default_rng(3)
    Wn, Tsub, D = 2, 188, 1024
    x0 = rng.standard_normal((Wn * Tsub, D)).astype(np.float32)

    def run_layer(c, use_fast=True):
        enc = fc.load_encoder(c, w)
        # drive the block directly from a given residual stream: reuse encode_batch's body through a
        # stand-in pre-encode (the subsampling front end is covered by the tiny end-to-end case)
        orig, orig_w = fc.pre_encode, fc.pre_encode_windows
        fc.pre_encode = lambda c_, e_, m_: (c_.upload(m_, Tsub, D), Tsub)
        fc.pre_encode_windows = lambda c_, e_, ms: (c_.upload(np.concatenate(ms), len(ms) * Tsub, D), Tsub)
        try:
            out, _ = fc.encode_batch(c, enc, [x0[i * Tsub:(i + 1) * Tsub] for i in range(Wn)], use_fast=use_fast)
        finally:
            fc.pre_encode, fc.pre_encode_windows = orig, orig_w
        return out

    ora = WasmOracle(threads=True)
    ref = run_layer(ora).array()
    h = ctx.pushArena()
    got = ctx.download(run_layer(ctx)).reshape(ref.shape)            # optional fast members (fused attention, ...)
    got_seq = ctx.download(run_layer(ctx, False)).reshape(ref.shape)  # the reference's exact op sequence
    ctx.popArena(h)
    assert np.abs(got - ref).max() <= 2e-2
    assert np.abs(got_seq - ref).max() <= 2e-2


def test_pipelined_encoder_returns_each_batch_in_order(ctx, pkg):
    """PipelinedEncoder (two recorded forwards on two streams, used alternately) hands back, one call late, exactly
    the frames encode_batch gives for the windows that were in the host buffers at submit time."""
    fc, synth = _eng()
    w = synth.encoder_weights(synth.TINY, seed=3)
    dev = ctx.device
    ctx, ctx2 = pkg.CudaContext(dev), pkg.CudaContext(dev)  # contexts of its own: recordings reserve pool blocks
    try:
        encs = [fc.load_encoder(ctx, w), fc.load_encoder(ctx2, w)]
        audio = synth.synth_audio(6, samples=16000 * 2, seed=4)
        mels = [fc.mel_time_major(synth.log_mel(a, 32).reshape(-1), 32) for a in audio]
        n = mels[0].size
        host = [[c.pinnedArray(n) for _ in range(2)] for c in (ctx, ctx2)]  # two windows per batch, per slot
        for bufs in host:
            for b, m in zip(bufs, mels[:2]):
                b[:] = m
        pipe = fc.PipelinedEncoder([ctx, ctx2], encs, lambda s: host[s], n)
        want = []
        got = []
        for step in range(3):
            pair = mels[2 * step:2 * step + 2]
            for b, m in zip(host[step % 2], pair):
                b[:] = m
            h = ctx.pushArena()
            ref, _ = fc.encode_batch(ctx, encs[0], [ctx.upload(m, 1, n) for m in pair])
            want.append(ctx.download(ref))
            ctx.popArena(h)
            r = pipe.submit()
            if r is not None:
                got.append(r.copy())
        got += pipe.flush()
        pipe.free()
        assert len(got) == 3
        for g, r in zip(got, want):
            assert np.array_equal(g, r)
    finally:
        ctx.destroy()
        ctx2.destroy()


def test_pipelined_encoder_post_op_rides_the_batch(ctx, pkg):
    """The `post` hook of PipelinedEncoder (the joint's encoder projection that the reference appends to the encoder's
    submission, src/engines/asr-parakeet/pipeline.js:57-61): what is read back is post(frames), identical to applying
    the same product to encode_batch's frames, and only its bytes cross to the host."""
    fc, synth = _eng()
    w = synth.encoder_weights(synth.TINY, seed=3)
    dev = ctx.device
    ctx, ctx2 = pkg.CudaContext(dev), pkg.CudaContext(dev)
    try:
        encs = [fc.load_encoder(ctx, w), fc.load_encoder(ctx2, w)]
        audio = synth.synth_audio(4, samples=16000 * 2, seed=5)
        mels = [fc.mel_time_major(synth.log_mel(a, 32).reshape(-1), 32) for a in audio]
        n = mels[0].size
        D = synth.TINY["D"]
        rng = np.random.default_rng(9)
        pw = (rng.standard_normal((D, 24)) / np.sqrt(D)).astype(np.float32)
        pb = rng.standard_normal(24).astype(np.float32)
        proj = [(c.uploadF16(pw, D, 24), c.upload(pb, 1, 24)) for c in (ctx, ctx2)]
        host = [[c.pinnedArray(n) for _ in range(2)] for c in (ctx, ctx2)]
        for bufs in host:
            for b, m in zip(bufs, mels[:2]):
                b[:] = m
        cs = (ctx, ctx2)
        pipe = fc.PipelinedEncoder([ctx, ctx2], encs, lambda s: host[s], n,
                                   post=lambda s, x: cs[s].matmul(x, proj[s][0], dict(bias=proj[s][1])))
        want, got = [], []
        for step in range(2):
            pair = mels[2 * step:2 * step + 2]
            for b, m in zip(host[step % 2], pair):
                b[:] = m
            h = ctx.pushArena()
            ref, _ = fc.encode_batch(ctx, encs[0], [ctx.upload(m, 1, n) for m in pair])
            want.append(ctx.download(ctx.matmul(ref, proj[0][0], dict(bias=proj[0][1]))))
            ctx.popArena(h)
            r = pipe.submit()
            if r is not None:
                got.append(r.copy())
        got += pipe.flush()
        pipe.free()
        assert len(got) == 2
        for g, r in zip(got, want):
            assert g.size == r.size and g.size % 24 == 0
            assert np.array_equal(g, r)
    finally:
        ctx.destroy()
        ctx2.destroy()


def test_int8_artifact_loader_resident_weights(ctx, pkg):
    """The encoder loaded from the int8 artifact (blob + manifest written by the restated quantiser) with the
    matrices kept int8 on the device: one full-width block, teacher-forced, against the oracle running the
    host-dequantised model (2e-2, the per-layer gate), and the tiny stack end to end against the f16-storage loader."""
    from fluidaudio_web_b200.engines import blob

    fc, synth = _eng()
    # tiny stack: int8-resident vs host-dequantised on the same backend
    w = synth.encoder_weights(synth.TINY, seed=3)
    data, man = blob.write_int8_blob(w)
    mels = [synth.log_mel(a, 32).reshape(-1) for a in synth.synth_audio(3, samples=16000 * 2, seed=3)]
    h = ctx.pushArena()
    a, _ = fc.encode_batch(ctx, fc.load_encoder_blob(ctx, data, man, int8_resident=True), mels)
    b, _ = fc.encode_batch(ctx, fc.load_encoder_blob(ctx, data, man, int8_resident=False), mels)
    assert np.abs(ctx.download(a) - ctx.download(b)).max() <= 2e-2
    ctx.popArena(h)
    # one real-size block
    cfg = dict(synth.PARAKEET_06B, layers=1)
    w = synth.encoder_weights(cfg, seed=3)
    data, man = blob.write_int8_blob(w)
    rng = np.random.default_rng(3)
    Wn, Tsub, D = 2, 188, 1024
    x0 = rng.standard_normal((Wn * Tsub, D)).astype(np.float32)

    def run_layer(c, enc):
        orig, orig_w = fc.pre_encode, fc.pre_encode_windows
        fc.pre_encode = lambda c_, e_, m_: (c_.upload(m_, Tsub, D), Tsub)
        fc.pre_encode_windows = lambda c_, e_, ms: (c_.upload(np.concatenate(ms), len(ms) * Tsub, D), Tsub)
        try:
            out, _ = fc.encode_batch(c, enc, [x0[i * Tsub:(i + 1) * Tsub] for i in range(Wn)])
        finally:
            fc.pre_encode, fc.pre_encode_windows = orig, orig_w
        return out

    ora = WasmOracle(threads=True)
    ref = run_layer(ora, fc.load_encoder_blob(ora, data, man)).array()  # the oracle has no resident-int8 member
    h = ctx.pushArena()
    enc = fc.load_encoder_blob(ctx, data, man, int8_resident=True)
    assert isinstance(enc["layers"][0]["ff1w1"], fc.Int8Weight) and isinstance(enc["layers"][0]["pw2T"], fc.Int8Weight)
    ctx.startProfile(512)
    got = ctx.download(run_layer(ctx, enc)).reshape(ref.shape)
    labels = {e["label"] for e in ctx.endProfile()}
    ctx.popArena(h)
    assert "tc_gemm_i8w_f16a" in labels and "tc_gemm_f16" not in labels  # every weight product ran on int8 weights
    assert np.abs(got - ref).max() <= 2e-2
