"""The int8 weight artifact (blob + manifest): writer against the reference quantiser's rules
(scripts/quantize-parakeet-encoder.py:20-59), reader against the loader's dequantisation
(src/engines/asr-parakeet/raw-encoder.js:56-76)."""
import json

import numpy as np


def _mods():
    import __graft_entry__ as ge

    ge.load_package()
    from fluidaudio_web_b200.engines import blob, synth

    return blob, synth


def test_layout_and_manifest_fields(tmp_path):
    blob, synth = _mods()
    w = synth.encoder_weights(synth.TINY, seed=3)
    data, man = blob.write_int8_blob(w)
    # f32 section first, then int8: every f32 offset (in floats) lies below the first int8 byte offset
    i8_base = min(m["i8ByteOffset"] for m in man.values() if m["dtype"] == "i8")
    for k, m in man.items():
        assert m["dims"] == list(w[k].shape) and m["count"] == w[k].size
        if m["dtype"] == "i8":
            assert m["quant"] == ("col" if (k == "linw" or k.split("_")[-1] in ("q", "k", "v", "pos", "out", "ff1w1", "ff1w2", "ff2w1", "ff2w2")) else "grp")
            assert m["scaleCount"] == (m["dims"][1] if m["quant"] == "col" else m["dims"][0])
            assert (m["scaleOffset"] + m["scaleCount"]) * 4 <= i8_base
        else:
            assert (m["offset"] + m["count"]) * 4 <= i8_base
    assert man["L0_lnff1_w"]["dtype"] == "f32" and man["c0b"]["dtype"] == "f32" and man["L1_dw"]["quant"] == "grp"
    assert len(data) == i8_base + sum(m["count"] for m in man.values() if m["dtype"] == "i8")
    blob.save(str(tmp_path / "weights.bin"), str(tmp_path / "manifest.json"), data, man)
    data2, man2 = blob.load(str(tmp_path / "weights.bin"), str(tmp_path / "manifest.json"))
    assert data2 == data and man2 == json.loads(json.dumps(man))


def test_reader_dequantises_like_the_loader():
    blob, synth = _mods()
    rng = np.random.default_rng(0)
    w = {"linw": rng.standard_normal((24, 10)).astype(np.float32), "c2w": rng.standard_normal((6, 6, 1, 1)).astype(np.float32),
         "L0_pw1": rng.standard_normal((8, 4, 1)).astype(np.float32), "L0_lnff1_w": rng.standard_normal(10).astype(np.float32),
         "L0_q": np.zeros((4, 3), np.float32)}
    data, man = blob.write_int8_blob(w)
    b = blob.Blob(data, man)
    q, sc, kind = b.tensor_i8("linw")
    assert kind == "col" and q.dtype == np.int8 and np.abs(q).max() == 127
    np.testing.assert_allclose(sc, np.abs(w["linw"]).max(0) / 127.0, rtol=1e-6)
    # out[i] = q[i] * sc[i % o]  (col)   /   q[i] * sc[i // rest]  (grp)
    flat = q.reshape(-1).astype(np.float32) * sc[np.arange(q.size) % 10]
    assert np.array_equal(b.tensor_f32("linw").reshape(-1), flat)
    q2, sc2, kind2 = b.tensor_i8("L0_pw1")
    assert kind2 == "grp"
    flat2 = q2.reshape(-1).astype(np.float32) * sc2[np.arange(q2.size) // 4]
    assert np.array_equal(b.tensor_f32("L0_pw1").reshape(-1), flat2)
    assert np.abs(b.tensor_f32("linw") - w["linw"]).max() <= np.abs(w["linw"]).max() / 127.0 * 0.5001
    assert np.array_equal(b.tensor_f32("L0_lnff1_w"), w["L0_lnff1_w"])
    assert np.array_equal(b.tensor_i8("L0_q")[1], np.ones(3, np.float32))  # all-zero columns get scale 1


def test_requantising_the_synthetic_weights_is_stable():
    """The synthetic encoder weights are dequantised int8 already: the artifact made from them dequantises to the same
    values to within one ulp of the scale, so the int8-resident and the host-dequantised loaders see the same model."""
    blob, synth = _mods()
    w = synth.encoder_weights(synth.TINY, seed=3)
    data, man = blob.write_int8_blob(w)
    b = blob.Blob(data, man)
    for k in w:
        assert np.abs(b.tensor_f32(k) - w[k]).max() <= 1e-6 * max(1.0, float(np.abs(w[k]).max()))
