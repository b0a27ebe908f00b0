"""The Whisper-shaped decoder engine run on the CPU oracle: the lock-step multi-stream driver must pick
the same tokens as the reference-form one-stream driver (raw-whisper-decoder.js:103-142), since both
compute the same per-row arithmetic."""
import numpy as np

import pytest

from oracle.wasm_oracle import WasmOracle


@pytest.fixture(autouse=True)
def _mods(pkg):
    global dec_mod, synth
    from fluidaudio_web_b200.engines import synth, whisper_decoder as dec_mod


def _setup(quant=None, S=3):
    cfg = synth.TINY_DEC
    ctx = WasmOracle()
    dec = dec_mod.load_decoder(ctx, synth.decoder_weights(cfg), cfg["NH"], quant=quant)
    encs = synth.encoder_states(cfg, S)
    return cfg, ctx, dec, encs


def test_infer_config_and_padding():
    cfg, ctx, dec, _ = _setup()
    c = dec["cfg"]
    assert (c["D"], c["FFN"], c["layers"], c["VOCAB"], c["HD"]) == (64, 128, 2, 203, 16)
    assert c["VOCABP"] == 204 and dec["embedT"].t.cols == 204
    assert np.all(dec["embedT"].t.array()[:, 203] == 0)


def test_streams_match_single_stream_on_oracle():
    for quant in (None, "int8"):
        cfg, ctx, dec, encs = _setup(quant)
        prefix, n_tok = [1, 2, 3, 4], 10
        single = []
        for s in range(len(encs)):
            enc = ctx.upload(encs[s], cfg["Tenc"], cfg["D"])
            single.append(dec_mod.greedy_decode(ctx, dec, enc, prefix, n_tok))
        enc_t = [ctx.upload(e, cfg["Tenc"], cfg["D"]) for e in encs]
        multi = dec_mod.greedy_decode_streams(ctx, dec, enc_t, prefix, n_tok)
        assert multi.tolist() == single
        assert len({tuple(r) for r in single}) > 1  # the clips really steer the tokens


def test_stream_logits_match_single_stream_logits():
    cfg, ctx, dec, encs = _setup()
    enc_t = [ctx.upload(e, cfg["Tenc"], cfg["D"]) for e in encs]
    kvS = dec_mod.cross_kv_streams(ctx, dec, enc_t)
    stS = dec_mod.decode_init_streams(ctx, dec, len(encs), 8)
    kv1 = dec_mod.cross_kv(ctx, dec, enc_t[1])
    st1 = dec_mod.decode_init(ctx, dec, 8)
    for tok in (5, 9, 100):
        _, lg = dec_mod.decode_next_streams(ctx, dec, kvS, stS, [tok] * len(encs), want_logits=True)
        ref = dec_mod.decode_next(ctx, dec, kv1, st1, tok)
        np.testing.assert_allclose(lg[1], ref, rtol=0, atol=1e-5)
