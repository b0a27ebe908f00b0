"""Whisper-shaped KV-cached greedy decoding on the CUDA backend against the same engine on the CPU
oracle: token ids must be identical (the reference's decode gate compares token ids between backends,
scripts/backend-parity.mjs; random-init logits are flat, so this is a strict test of the f32-grade
activation path that decode-size products take on the tensor cores).  The smallest top-2 logit margin
seen on the oracle is asserted to be far above the measured logit error, so identity is not luck."""
import numpy as np
import pytest

from oracle.wasm_oracle import WasmOracle

pytestmark = pytest.mark.gpu

MID = dict(D=256, NH=4, FFN=1024, layers=2, VOCAB=2003, maxPos=40, Tenc=96)


def _mods():
    from fluidaudio_web_b200.engines import synth, whisper_decoder

    return whisper_decoder, synth


def _oracle_tokens(dm, synth, cfg, w, encs, prefix, n_tok, quant, margins):
    ora = WasmOracle(threads=True)
    dec = dm.load_decoder(ora, w, cfg["NH"], quant=quant)
    return [dm.greedy_decode(ora, dec, ora.upload(e, cfg["Tenc"], cfg["D"]), prefix, n_tok, margins) for e in encs]


@pytest.mark.parametrize("quant", [None, "int8"])
@pytest.mark.parametrize("cfg_name,S,n_tok", [("tiny", 3, 10), ("mid", 32, 12)])
def test_stream_tokens_identical_to_oracle(ctx, pkg, cfg_name, S, n_tok, quant):
    dm, synth = _mods()
    cfg = synth.TINY_DEC if cfg_name == "tiny" else MID
    w = synth.decoder_weights(cfg, seed=11)
    encs = synth.encoder_states(cfg, S, seed=13)
    prefix = [1, 2, 3, 4]
    margins = []
    want = _oracle_tokens(dm, synth, cfg, w, encs, prefix, n_tok, quant, margins)
    ctx.setOption("int8_limbs", 3)  # f32-grade int8 activations, like the f16 value+residue planes
    ctx.setOption("f16_hilo_rows", 1 << 30)  # ... for the many-row cross K/V products as well
    h = ctx.pushArena()
    try:
        dec = dm.load_decoder(ctx, w, cfg["NH"], quant=quant)
        enc_t = [ctx.upload(e, cfg["Tenc"], cfg["D"]) for e in encs]
        got = dm.greedy_decode_streams(ctx, dec, enc_t, prefix, n_tok)
        # one-stream reference-form driver on the device as well (stream 0)
        got0 = dm.greedy_decode(ctx, dec, enc_t[0], prefix, n_tok)
    finally:
        ctx.popArena(h)
        ctx.setOption("int8_limbs", 2)
        ctx.setOption("f16_hilo_rows", 64)
    assert got.tolist() == want, f"min oracle top-2 margin {min(margins):.3e}"
    assert got0 == want[0]


def test_stream_logits_close_and_margin(ctx, pkg):
    """Logit error of the lock-step device path against the oracle, next to the oracle's top-2 margins."""
    dm, synth = _mods()
    cfg, S = MID, 32
    w = synth.decoder_weights(cfg, seed=11)
    encs = synth.encoder_states(cfg, S, seed=13)
    ora = WasmOracle(threads=True)
    dec_o = dm.load_decoder(ora, w, cfg["NH"])
    kv_o = dm.cross_kv_streams(ora, dec_o, [ora.upload(e, cfg["Tenc"], cfg["D"]) for e in encs])
    st_o = dm.decode_init_streams(ora, dec_o, S, 8)
    ctx.setOption("f16_hilo_rows", 1 << 30)
    h = ctx.pushArena()
    try:
        dec = dm.load_decoder(ctx, w, cfg["NH"])
        kv = dm.cross_kv_streams(ctx, dec, [ctx.upload(e, cfg["Tenc"], cfg["D"]) for e in encs])
        st = dm.decode_init_streams(ctx, dec, S, 8)
        toks = np.arange(S) % 7 + 1
        for _ in range(4):
            nxt_o, lg_o = dm.decode_next_streams(ora, dec_o, kv_o, st_o, toks, want_logits=True)
            nxt, lg = dm.decode_next_streams(ctx, dec, kv, st, toks, want_logits=True)
            err = float(np.abs(lg - lg_o).max())
            top2 = np.sort(lg_o, axis=1)[:, -2:]
            margin = float((top2[:, 1] - top2[:, 0]).min())
            assert err <= 2e-5, err  # logits are O(1): f32-grade, not f16-grade (which is ~1e-3 here)
            assert np.array_equal(nxt, nxt_o) or margin < 10 * err
            toks = nxt_o
    finally:
        ctx.popArena(h)
        ctx.setOption("f16_hilo_rows", 64)


def test_full_width_steps_match_oracle(ctx, pkg):
    """large-v3-turbo widths (D 1280, 20 heads, FFN 5120, vocab 51866 -> 51868) with a short encoder
    sequence so the CPU side stays in seconds: 4 streams, 3 lock-step tokens, f16 and int8 weights."""
    dm, synth = _mods()
    cfg = dict(synth.WHISPER_TURBO_DEC, layers=2, Tenc=48, maxPos=8)
    S = 4
    w = synth.decoder_weights(cfg, seed=17)
    encs = synth.encoder_states(cfg, S, seed=19)
    for quant in (None, "int8"):
        ora = WasmOracle(threads=True)
        dec_o = dm.load_decoder(ora, w, cfg["NH"], quant=quant)
        kv_o = dm.cross_kv_streams(ora, dec_o, [ora.upload(e, cfg["Tenc"], cfg["D"]) for e in encs])
        st_o = dm.decode_init_streams(ora, dec_o, S, 4)
        ctx.setOption("int8_limbs", 3)
        ctx.setOption("f16_hilo_rows", 1 << 30)
        h = ctx.pushArena()
        try:
            dec = dm.load_decoder(ctx, w, cfg["NH"], quant=quant)
            assert dec["cfg"]["VOCABP"] == 51868
            kv = dm.cross_kv_streams(ctx, dec, [ctx.upload(e, cfg["Tenc"], cfg["D"]) for e in encs])
            st = dm.decode_init_streams(ctx, dec, S, 4)
            toks = np.array([1, 2, 3, 4])
            for _ in range(3):
                nxt_o, lg_o = dm.decode_next_streams(ora, dec_o, kv_o, st_o, toks, want_logits=True)
                nxt, lg = dm.decode_next_streams(ctx, dec, kv, st, toks, want_logits=True)
                assert lg.shape == (S, 51866)
                err = float(np.abs(lg - lg_o).max())
                top2 = np.sort(lg_o, axis=1)[:, -2:]
                margin = float((top2[:, 1] - top2[:, 0]).min())
                assert err <= 5e-5, (quant, err)
                assert np.array_equal(nxt, nxt_o) or margin < 10 * err, (quant, err, margin)
                toks = nxt_o
        finally:
            ctx.popArena(h)
            ctx.setOption("int8_limbs", 2)
            ctx.setOption("f16_hilo_rows", 64)


def test_resident_loop_and_recorded_replay_match_oracle(ctx, pkg):
    """The greedy loop with token pick and embedding gather on the device (no host round trip), eager and
    as one recorded batch replayed twice, picks the oracle's tokens."""
    dm, synth = _mods()
    cfg, S, n_tok = MID, 32, 12
    w = synth.decoder_weights(cfg, seed=11)
    encs = synth.encoder_states(cfg, S, seed=13)
    prefix = [1, 2, 3, 4]
    want = _oracle_tokens(dm, synth, cfg, w, encs, prefix, n_tok, None, [])
    ctx.setOption("f16_hilo_rows", 1 << 30)
    h = ctx.pushArena()
    try:
        dec = dm.load_decoder(ctx, w, cfg["NH"])
        dm.resident_tables(ctx, dec)
        enc_all = ctx.upload(encs.reshape(S * cfg["Tenc"], cfg["D"]), S * cfg["Tenc"], cfg["D"])
        pidx = [ctx.upload(np.full(S, t, np.float32), S, 1) for t in prefix]
        st = dm.decode_init_streams(ctx, dec, S, len(prefix) + n_tok)
        run = lambda: dm.greedy_decode_streams_resident(ctx, dec, enc_all, S, pidx, n_tok, st=st)
        hist = run()
        got = ctx.download(hist).reshape(n_tok, S).T.astype(np.int64)
        assert got.tolist() == want
        batch, hist2 = ctx.recordBatch(run)
        for _ in range(2):
            batch.launch()
            got2 = ctx.download(hist2).reshape(n_tok, S).T.astype(np.int64)
            assert got2.tolist() == want
        batch.free()
    finally:
        ctx.popArena(h)
        ctx.setOption("f16_hilo_rows", 64)


def test_embed_rows_and_bad_token(ctx, pkg):
    rng = np.random.default_rng(3)
    table = rng.standard_normal((50, 96)).astype(np.float32)
    pos = rng.standard_normal((10, 96)).astype(np.float32)
    ids = np.array([[3, 0.5], [49, 1.0], [0, -2.0]], np.float32)  # argmax-shaped [S,2]
    t, p, i = ctx.upload(table, 50, 96), ctx.upload(pos, 10, 96), ctx.upload(ids, 3, 2)
    got = ctx.download(ctx.embedRows(t, p, i, 7)).reshape(3, 96)
    assert np.array_equal(got, table[[3, 49, 0]] + pos[7][None, :])
    with pytest.raises(Exception):
        ctx.embedRows(t, p, i, 10)  # position outside the table
    bad = ctx.upload(np.array([[50.0]], np.float32), 1, 1)
    ctx.embedRows(t, p, bad, 0)
    with pytest.raises(Exception, match="token id"):
        ctx.sync()
    ctx.sync()  # the flag is cleared once reported


@pytest.mark.parametrize("W,H,HD,Tk", [(1, 4, 16, 7), (3, 8, 64, 131), (1, 96, 64, 33), (5, 2, 128, 70), (2, 3, 20, 9)])
def test_single_query_attention_products(ctx, pkg, W, H, HD, Tk):
    """bmmQK / bmmPV with one query row per window (the decode-step form) against the oracle."""
    ora = WasmOracle()
    rng = np.random.default_rng(W * 100 + H)
    S = H * HD
    q = rng.standard_normal((W, S)).astype(np.float32)
    k = rng.standard_normal((W * Tk, S)).astype(np.float32)
    qb = rng.standard_normal((1, S)).astype(np.float32)
    for shared in (False, True):
        kk = k[:Tk] if shared else k
        ref = ora.bmmQK(ora.upload(q, W, S), ora.upload(kk, kk.shape[0], S), ora.upload(qb, 1, S), H, HD, W, shared).array()
        got = ctx.download(ctx.bmmQK(ctx.upload(q, W, S), ctx.upload(kk, kk.shape[0], S), ctx.upload(qb, 1, S), H, HD, W, shared))
        np.testing.assert_allclose(got.reshape(ref.shape), ref, rtol=0, atol=2e-5 * np.sqrt(HD))
    p = rng.random((W * H, Tk)).astype(np.float32)
    ref = ora.bmmPV(ora.upload(p, W * H, Tk), ora.upload(k, W * Tk, S), H, HD, W).array()
    got = ctx.download(ctx.bmmPV(ctx.upload(p, W * H, Tk), ctx.upload(k, W * Tk, S), H, HD, W))
    np.testing.assert_allclose(got.reshape(ref.shape), ref, rtol=0, atol=2e-5 * np.sqrt(Tk))


@pytest.mark.parametrize("M,K,N", [(1, 1280, 5120), (4, 5120, 1280), (64, 1280, 1290), (33, 200, 640)])
def test_few_row_f16_products_are_f32_grade(ctx, pkg, M, K, N):
    """Products with <= 64 rows feed the tensor cores value+residue planes: the result tracks the f32
    oracle ~1000x closer than single-plane f16 activations would (whose error here is ~1e-3)."""
    ora = WasmOracle(threads=True)
    rng = np.random.default_rng(M + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    ref = ora.matmul(ora.upload(a, M, K), ora.upload(b, K, N), dict(bias=ora.upload(bias, 1, N), act="gelu_erf")).array()
    got = ctx.download(ctx.matmul(ctx.upload(a, M, K), ctx.uploadF16(b, K, N), dict(bias=ctx.upload(bias, 1, N), act="gelu_erf")))
    assert np.abs(got.reshape(ref.shape) - ref).max() <= 2e-5
