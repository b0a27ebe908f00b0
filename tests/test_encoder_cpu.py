"""Host-side logic of the FastConformer engine, run on the CPU oracle backend (no GPU): shapes, the
positional table, weight folding, and that the forward is a pure function of seeded inputs."""
import numpy as np

from oracle.wasm_oracle import WasmOracle


def _eng(pkg):
    from fluidaudio_web_b200.engines import fastconformer, synth

    return fastconformer, synth


def test_infer_config_and_shapes(pkg):
    fc, synth = _eng(pkg)
    w = synth.encoder_weights(synth.TINY, seed=3)
    cfg = fc.infer_config(w)
    assert {k: cfg[k] for k in ("D", "DFF", "H", "HD", "layers", "dwK", "Csub", "melBins")} == synth.TINY
    ora = WasmOracle(threads=True)
    enc = fc.load_encoder(ora, w)
    mels = [synth.log_mel(a, 32) for a in synth.synth_audio(2, samples=16000 * 2, seed=3)]
    assert mels[0].shape == (32, 201)
    x, Tsub = fc.encode_batch(ora, enc, [m.reshape(-1) for m in mels])
    assert Tsub == 26 and (x.rows, x.cols) == (2 * 26, 64)
    assert np.isfinite(x.array()).all()
    # windows are independent: encoding window 1 alone gives the same frames as inside the batch
    x1, _ = fc.encode_batch(ora, fc.load_encoder(ora, w), [mels[1].reshape(-1)])
    assert np.abs(x.array()[26:] - x1.array()).max() < 1e-4


def test_pos_encoding_matches_definition(pkg):
    fc, _ = _eng(pkg)
    pe = fc.pos_encoding(5, 8)
    assert pe.shape == (9, 8)
    assert np.allclose(pe[4], np.tile([0, 1], 4))  # position 0: sin 0, cos 0
    assert np.isclose(pe[0, 0], np.sin(4.0)) and np.isclose(pe[8, 1], np.cos(-4.0))


def test_quantiser_roundtrip_is_int8_grid(pkg):
    _, synth = _eng(pkg)
    w = synth.encoder_weights(synth.TINY, seed=3)["L0_ff1w1"]
    scale = np.abs(w).max(0) / 127.0
    q = w / scale
    assert np.abs(q - np.round(q)).max() < 1e-3 and np.abs(q).max() <= 127.001


def test_mel_front_end_is_normalised(pkg):
    _, synth = _eng(pkg)
    m = synth.log_mel(synth.synth_audio(1, samples=240000, seed=3)[0], 128)
    assert m.shape == (128, 1501)
    assert np.abs(m.mean(1)).max() < 1e-3 and np.abs(m.std(1, ddof=1) - 1).max() < 1e-2
