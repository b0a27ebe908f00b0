"""The C restatement of the reference's log-mel front end (oracle/nemo_mel_port.c) against an independent
formulation of the same pipeline (numpy rfft over explicitly framed, windowed samples) - the known-answer material
for this part: the reference's own code is plain JavaScript and cannot run here."""
import numpy as np

from oracle.mel_oracle import filterbank, nemotron_mel, parakeet_mel, raw_mel


def _independent_raw(audio, n_mels, guard):
    x = audio.astype(np.float32)
    pre = (x[1:].astype(np.float64) - 0.97 * x[:-1].astype(np.float64)).astype(np.float32)
    x = np.pad(np.concatenate([x[:1], pre]).astype(np.float64), 256)
    T = 1 + (x.size - 512) // 160
    win = np.zeros(512)
    win[56:456] = 0.5 - 0.5 * np.cos(2 * np.pi * np.arange(400) / 399)
    idx = np.arange(512)[None, :] + 160 * np.arange(T)[:, None]
    spec = np.fft.rfft(x[idx] * win, axis=1)
    power = (spec.real ** 2 + spec.imag ** 2).astype(np.float32)
    fb, _ = filterbank(n_mels)
    return np.log(power.astype(np.float64) @ fb.astype(np.float64).T + guard).T.astype(np.float32)


def _audio(n, seed):
    rng = np.random.default_rng(seed)
    t = np.arange(n) / 16000.0
    return (0.1 * rng.standard_normal(n) + 0.3 * np.sin(2 * np.pi * 440 * t) + 0.05 * np.sin(2 * np.pi * 3100 * t)).astype(np.float32)


def test_raw_log_mel_matches_rfft_formulation():
    for n, n_mels in ((16000, 128), (4000, 80), (163, 128)):
        a = _audio(n, n)
        raw, feat = raw_mel(a, n_mels, 2.0 ** -24)
        assert raw.shape == (n_mels, n // 160 + 1) and feat == n // 160
        ref = _independent_raw(a, n_mels, 2.0 ** -24)
        assert np.abs(raw - ref).max() <= 2e-5  # f32 logs of doubles that differ in summation order only


def test_filterbank_rows_are_slaney_triangles():
    fb, bounds = filterbank(128)
    assert fb.shape == (128, 257) and (fb >= 0).all()
    for m in range(128):
        nz = np.nonzero(fb[m])[0]
        assert nz.size and bounds[m, 0] == nz[0] and bounds[m, 1] == nz[-1] + 1
        peak = int(np.argmax(fb[m]))
        assert (np.diff(fb[m, nz[0]:peak + 1]) >= 0).all() and (np.diff(fb[m, peak:nz[-1] + 1]) <= 0).all()
    # slaney norm: every triangle integrates to one over frequency (bins are 31.25 Hz apart; the narrow low filters
    # span two or three bins, so their sampled area is coarse)
    area = fb.sum(1) * (8000.0 / 256)
    assert np.abs(area - 1.0).max() < 0.35 and np.abs(area[100:] - 1.0).max() < 0.03


def test_parakeet_normalisation_and_nemotron_raw():
    a = _audio(24000, 3)
    f = parakeet_mel(a)
    assert f.shape == (128, 150)
    assert np.abs(f.mean(1)).max() < 1e-4
    assert np.abs(f.std(1, ddof=1) - 1.0).max() < 1e-3
    r = nemotron_mel(a)
    assert r.shape == (128, 151) and np.isfinite(r).all()
    silent = parakeet_mel(np.zeros(1600, np.float32))
    assert np.allclose(silent, 0.0)  # constant rows: (x - mean) = 0
