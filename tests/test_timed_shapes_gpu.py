"""Parity at the shapes the benchmark times (the other GPU tests use small shapes so the oracle is quick).

Rows of a matrix product are independent, so the CPU oracle run on a sample of the rows of A prices a
16384-row check at seconds and is exact for those rows.  Tolerances are the reference gate's
(scripts/backend-conformance.mjs:67-141): 2e-2 max-abs on unit-scale outputs for the f16-weight route,
1e-3 relative for int8; greedy token ids identical.
"""
import numpy as np
import pytest

from oracle.wasm_oracle import T, WasmOracle

pytestmark = pytest.mark.gpu

W_WINDOWS, TSUB, D, DFF = 32, 188, 1024, 4096
M_BLOCK = W_WINDOWS * TSUB  # 6016 rows: the encoder batch the benchmark runs


def _sample_rows(M, n=64, seed=0):
    rng = np.random.default_rng(seed)
    rows = np.unique(np.concatenate([[0, 1, M - 2, M - 1], rng.integers(0, M, n)]))
    return rows[:n]


def _check_product(ctx, M, K, N, *, bias=False, act="none", add=False, operand_only=False, seed=0):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)  # both sides see f16 weights
    b = rng.standard_normal(N).astype(np.float32) if bias else None
    r = rng.standard_normal((M, N)).astype(np.float32) if add else None
    h = ctx.pushArena()
    try:
        opts = dict(act=act)
        if bias:
            opts["bias"] = ctx.upload(b, 1, N)
        if add:
            opts["add"] = ctx.upload(r, M, N)
        if operand_only:
            opts["operandOnly"] = True
        wt = ctx.uploadF16(w, K, N)
        got = ctx.download(ctx.matmul(ctx.upload(a, M, K), wt, opts)).reshape(M, N)
        ctx.freeTensor(wt)
    finally:
        ctx.popArena(h)
    rows = _sample_rows(M, seed=seed)
    ora = WasmOracle(threads=True)
    ref = ora.matmul(T(a[rows], len(rows), K), T(w, K, N), bias=T(b, 1, N) if bias else None, act=act,
                     add=T(r[rows], len(rows), N) if add else None).array()
    err = float(np.abs(got[rows] - ref).max())
    assert err <= 2e-2, f"M={M} K={K} N={N} act={act}: max abs err {err}"
    return err


BLOCK_PRODUCTS = [
    ("ff_up_silu", D, DFF, dict(bias=True, act="silu")),
    ("ff_down_residual", DFF, D, dict(bias=True, add=True)),
    ("qkv_fused_operand", D, 3 * D, dict(bias=True, operand_only=True)),
    ("out_proj_residual", D, D, dict(bias=True, add=True)),
    ("pointwise1", D, 2 * D, dict(bias=True)),
]


@pytest.mark.parametrize("name,K,N,kw", BLOCK_PRODUCTS, ids=[b[0] for b in BLOCK_PRODUCTS])
def test_conformer_block_products_at_benchmark_rows(ctx, name, K, N, kw):
    _check_product(ctx, M_BLOCK, K, N, seed=len(name), **kw)


@pytest.mark.parametrize("M", [4096, 16384])
@pytest.mark.parametrize("K,N", [(1024, 3072), (1024, 1024), (1024, 4096), (4096, 1024)])
def test_f16_sweep_large_rows(ctx, M, K, N):
    _check_product(ctx, M, K, N, seed=M + N)


def test_f16_sweep_epilogue_at_16384_rows(ctx):
    _check_product(ctx, 16384, 1024, 4096, bias=True, act="silu", seed=5)
    _check_product(ctx, 16384, 4096, 1024, bias=True, add=True, seed=6)


def test_int8_gemm_benchmark_shape_sampled_rows(ctx):
    """512 x 1024 x 4096 against the oracle in the reference's own loop order on 64 rows."""
    rng = np.random.default_rng(0)
    M, K, N = 512, 1024, 4096
    a = rng.standard_normal((M, K)).astype(np.float32)
    wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    sc = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
    y = ctx.download(ctx.matmulInt8(ctx.upload(a, M, K), ctx.uploadBytes(wq), ctx.upload(sc, 1, N), N, K)).reshape(M, N)
    rows = _sample_rows(M, seed=1)
    ora = WasmOracle(threads=True)
    ref = ora.matmulInt8(T(a[rows], len(rows), K), ora.uploadBytes(wq), T(sc, 1, N), N, K).array()
    rms = np.sqrt((ref.astype(np.float64) ** 2).mean())
    assert float((np.abs(y[rows] - ref) / np.maximum(np.abs(ref), rms)).max()) <= 1e-3


@pytest.mark.parametrize("N", [2048, 8192])
@pytest.mark.parametrize("M", [1, 4, 16])
def test_int4_decode_benchmark_shapes(ctx, M, N):
    rng = np.random.default_rng(1)
    K = 2048
    nblk = K // 32
    a = rng.standard_normal((M, K)).astype(np.float16).astype(np.float32)
    bq = rng.integers(0, 256, N * nblk * 16, dtype=np.uint8)
    scales = rng.uniform(5e-3, 2e-2, N * nblk).astype(np.float16).astype(np.float32)
    zp = np.full(N * (nblk // 2), 0x88, np.uint8)
    got = ctx.download(ctx.matmulNBits(ctx.upload(a, M, K), ctx.uploadBytes(bq), ctx.upload(scales, 1, scales.size),
                                       ctx.uploadBytes(zp), N)).reshape(M, N)
    ora = WasmOracle(threads=True)
    ref = ora.matmulNBits(T(a, M, K), ora.uploadBytes(bq), T(scales, 1, scales.size), ora.uploadBytes(zp), N).array()
    assert float(np.abs(got - ref).max()) <= 2e-2  # outputs ~ N(0, 2.6): unit scale


def test_full_stack_layer_report(ctx, pkg, capsys):
    """The 24-layer, full-width encoder on two 15 s windows.  Gate: every layer, teacher-forced (fed the oracle's
    input for that layer), within 2e-2 of the oracle's output.  Report (printed, no gate): drift of the free-running
    stack against the oracle after each layer - random-init stacks amplify rounding layer over layer."""
    from fluidaudio_web_b200.engines import fastconformer as fc, synth

    cfg = dict(synth.PARAKEET_06B)
    w = synth.encoder_weights(cfg, seed=3)
    mels = [synth.log_mel(a, 128).reshape(-1) for a in synth.synth_audio(2, seed=3)]
    ora = WasmOracle(threads=True)
    ref_layers = []
    ref_pre = {}

    enc_o = fc.load_encoder(ora, w)
    orig_pre = fc.pre_encode

    def pre_capture(c_, e_, m_):
        x, t = orig_pre(c_, e_, m_)
        if c_ is ora:
            ref_pre.setdefault("x", []).append(x.array().copy())
        return x, t

    fc.pre_encode = pre_capture
    try:
        fc.encode_batch(ora, enc_o, mels, layer_hook=lambda L, x: ref_layers.append(x.array().copy()))
    finally:
        fc.pre_encode = orig_pre
    x0 = np.concatenate(ref_pre["x"])  # oracle's front-end output [2*188, 1024]
    assert len(ref_layers) == cfg["layers"] and x0.shape == (2 * TSUB, D)

    enc = fc.load_encoder(ctx, w)
    got_layers = []
    h = ctx.pushArena()
    try:
        got, tsub = fc.encode_batch(ctx, enc, mels, layer_hook=lambda L, x: got_layers.append(ctx.download(x).reshape(-1, D)))
        assert tsub == TSUB
        front = None
    finally:
        ctx.popArena(h)

    # teacher-forced: layer L alone from the oracle's input to it
    orig, orig_w = fc.pre_encode, fc.pre_encode_windows
    forced = []
    try:
        for L in range(cfg["layers"]):
            xin = x0 if L == 0 else ref_layers[L - 1]
            fc.pre_encode = lambda c_, e_, m_: (c_.upload(m_, TSUB, D), TSUB)
            fc.pre_encode_windows = lambda c_, e_, ms: (c_.upload(np.concatenate(ms), len(ms) * TSUB, D), TSUB)
            one = dict(enc, layers=[enc["layers"][L]], cfg=dict(enc["cfg"], layers=1), _posProj={})
            h = ctx.pushArena()
            out, _ = fc.encode_batch(ctx, one, [xin[:TSUB], xin[TSUB:]])
            forced.append(float(np.abs(ctx.download(out).reshape(-1, D) - ref_layers[L]).max()))
            ctx.popArena(h)
    finally:
        fc.pre_encode, fc.pre_encode_windows = orig, orig_w

    lines = ["layer  teacher-forced max|d|   free-running max|d|   free-running rms(d)"]
    for L in range(cfg["layers"]):
        d = got_layers[L] - ref_layers[L]
        lines.append(f"{L:5d}  {forced[L]:20.3e}  {np.abs(d).max():20.3e}  {np.sqrt((d ** 2).mean()):20.3e}")
    with capsys.disabled():
        print("\n[full-stack encoder report, 2 windows x 188 frames, D=1024]\n" + "\n".join(lines))
    assert max(forced) <= 2e-2, f"teacher-forced per-layer errors: {forced}"
    assert np.isfinite(got_layers[-1]).all()


@pytest.mark.parametrize("quant,n_check", [(None, 4), ("int8", 2)])
def test_decoder_config_token_identity_sampled_streams(ctx, pkg, quant, n_check):
    """64 concurrent greedy streams of 224 tokens (4-token forced prefix, Tenc 1500, large-v3-turbo widths) on the
    device; a sample of the streams is decoded by the oracle over all 224 tokens and must match id for id."""
    from fluidaudio_web_b200.engines import synth, whisper_decoder as dm

    cfg = dict(synth.WHISPER_TURBO_DEC, Tenc=1500)
    S, n_tok, prefix = 64, 224, [1, 2, 3, 4]
    w = synth.decoder_weights(cfg, seed=5)
    encs = synth.encoder_states(cfg, S, seed=7)  # one clip per stream
    ctx.setOption("int8_limbs", 3)
    ctx.setOption("f16_hilo_rows", 1 << 30)
    h = ctx.pushArena()
    try:
        dec = dm.load_decoder(ctx, w, cfg["NH"], quant=quant)
        enc_all = ctx.upload(np.ascontiguousarray(encs).reshape(S * cfg["Tenc"], cfg["D"]), S * cfg["Tenc"], cfg["D"])
        prefix_idx = [ctx.upload(np.full(S, t, np.float32), S, 1) for t in prefix]
        hist = dm.greedy_decode_streams_resident(ctx, dec, enc_all, S, prefix_idx, n_tok)
        got = ctx.download(hist).reshape(n_tok, S).T.astype(np.int64)  # [S, n_tok]
    finally:
        ctx.popArena(h)
        ctx.setOption("int8_limbs", 2)
        ctx.setOption("f16_hilo_rows", 64)
    ora = WasmOracle(threads=True)
    dec_o = dm.load_decoder(ora, w, cfg["NH"], quant=quant)
    picks = [0, 63, 21, 42][:n_check]
    for s in picks:
        margins = []
        want = dm.greedy_decode(ora, dec_o, ora.upload(encs[s], cfg["Tenc"], cfg["D"]), prefix, n_tok, margins)
        assert got[s].tolist() == list(want), f"stream {s} ({quant}): first mismatch at token " \
            f"{int(np.argmax(got[s] != np.array(want)))}, min oracle top-2 margin {min(margins):.3e}"
