"""Seeded synthetic stand-ins for the benchmark inputs of the FastConformer encoder: random-init
weights in the reference manifest's naming and shapes, quantised int8 with the reference quantiser
(scripts/quantize-parakeet-encoder.py:31-42) and dequantised the way the loader does
(src/engines/asr-parakeet/raw-encoder.js:55-76); synthetic audio; and the NeMo log-mel front-end
(src/engines/asr-nemotron/nemotron-mel.js, Parakeet settings of src/engines/asr-parakeet/parakeet-mel.js).
No real speech or checkpoint is involved."""
from __future__ import annotations

import math
from typing import Dict

import numpy as np

PARAKEET_06B = dict(D=1024, DFF=4096, H=8, HD=128, layers=24, dwK=9, Csub=256, melBins=128)
TINY = dict(D=64, DFF=128, H=4, HD=16, layers=2, dwK=9, Csub=8, melBins=32)


def _quant_cols(a: np.ndarray) -> np.ndarray:
    """Per-output-column int8 (matrices [in, out]) -> dequantised f32 (quantize-parakeet-encoder.py:31-36)."""
    scale = np.abs(a).max(0) / 127.0
    scale[scale == 0] = 1
    q = np.clip(np.round(a / scale), -127, 127).astype(np.int8)
    return (q.astype(np.float32) * scale.astype(np.float32)).astype(np.float32)


def _quant_rows(a: np.ndarray) -> np.ndarray:
    """Per-Cout int8 for conv weights (:37-42)."""
    a2 = a.reshape(a.shape[0], -1)
    scale = np.abs(a2).max(1) / 127.0
    scale[scale == 0] = 1
    q = np.clip(np.round(a2 / scale[:, None]), -127, 127).astype(np.int8)
    return (q.astype(np.float32) * scale[:, None].astype(np.float32)).astype(np.float32).reshape(a.shape)


def encoder_weights(cfg: dict, seed: int = 3) -> Dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    D, DFF, H, HD, Csub = cfg["D"], cfg["DFF"], cfg["H"], cfg["HD"], cfg["Csub"]
    Fsub = cfg["melBins"] // 8
    n = lambda shape, fan_in: (rng.standard_normal(shape) / math.sqrt(fan_in)).astype(np.float32)
    w: Dict[str, np.ndarray] = {}
    w["c0w"] = _quant_rows(n((Csub, 1, 3, 3), 9))
    w["c1w"] = _quant_rows(n((Csub, 1, 3, 3), 9))
    w["c2w"] = _quant_rows(n((Csub, Csub, 1, 1), Csub))
    w["c3w"] = _quant_rows(n((Csub, 1, 3, 3), 9))
    w["c4w"] = _quant_rows(n((Csub, Csub, 1, 1), Csub))
    for i in range(5):
        w[f"c{i}b"] = (rng.standard_normal(Csub) * 0.02).astype(np.float32)
    w["linw"] = _quant_cols(n((Csub * Fsub, D), Csub * Fsub))
    w["linb"] = (rng.standard_normal(D) * 0.02).astype(np.float32)
    for L in range(cfg["layers"]):
        g = lambda s: f"L{L}_{s}"
        for nm in ("lnff1", "lnatt", "lnconv", "lnff2", "lnout"):
            w[g(nm + "_w")] = np.ones(D, np.float32)
            w[g(nm + "_b")] = np.zeros(D, np.float32)
        w[g("ff1w1")] = _quant_cols(n((D, DFF), D))
        w[g("ff1w2")] = _quant_cols(n((DFF, D), DFF))
        w[g("ff2w1")] = _quant_cols(n((D, DFF), D))
        w[g("ff2w2")] = _quant_cols(n((DFF, D), DFF))
        for nm in ("q", "k", "v", "pos", "out"):
            w[g(nm)] = _quant_cols(n((D, D), D))
        w[g("pbu")] = (rng.standard_normal((H, HD)) * 0.02).astype(np.float32)
        w[g("pbv")] = (rng.standard_normal((H, HD)) * 0.02).astype(np.float32)
        w[g("pw1")] = _quant_rows(n((2 * D, D, 1), D))
        w[g("dw")] = _quant_rows(n((D, 1, cfg["dwK"]), cfg["dwK"]))
        w[g("dwb")] = (rng.standard_normal(D) * 0.02).astype(np.float32)
        w[g("pw2")] = _quant_rows(n((D, D, 1), D))
    return w


WHISPER_TURBO_DEC = dict(D=1280, NH=20, FFN=5120, layers=4, VOCAB=51866, maxPos=448, Tenc=1500)
TINY_DEC = dict(D=64, NH=4, FFN=128, layers=2, VOCAB=203, maxPos=40, Tenc=24)


def decoder_weights(cfg: dict, seed: int = 5) -> Dict[str, np.ndarray]:
    """Random-init weights in the naming and shapes of the Whisper decoder manifest
    (src/engines/asr-whisper/raw-whisper-decoder.js:33-56, embed/pos/lnf :66-71).  Matrix values are
    f16-representable (the artifact's f16 variant), so f16 storage loses nothing against f32 storage."""
    rng = np.random.default_rng(seed)
    D, FFN = cfg["D"], cfg["FFN"]
    h16 = lambda a: a.astype(np.float16).astype(np.float32)
    n = lambda shape, fan_in: h16(rng.standard_normal(shape, dtype=np.float32) / np.float32(math.sqrt(fan_in)))
    small = lambda m: (rng.standard_normal(m) * 0.02).astype(np.float32)
    w: Dict[str, np.ndarray] = {}
    for L in range(cfg["layers"]):
        g = lambda s: f"L{L}_{s}"
        for nm in ("sqw", "skw", "svw", "sow", "cqw", "ckw", "cvw", "cow"):
            w[g(nm)] = n((D, D), D)
        for nm in ("sqb", "svb", "sob", "cqb", "cvb", "cob", "f2b"):
            w[g(nm)] = small(D)
        w[g("f1w")] = n((D, FFN), D)
        w[g("f1b")] = small(FFN)
        w[g("f2w")] = n((FFN, D), FFN)
        for nm in ("ln1", "ln2", "ln3"):
            w[g(nm + "w")] = (1.0 + rng.standard_normal(D) * 0.05).astype(np.float32)
            w[g(nm + "b")] = small(D)
    w["embed"] = h16(rng.standard_normal((cfg["VOCAB"], D), dtype=np.float32) * np.float32(0.05))
    w["pos"] = (rng.standard_normal((cfg["maxPos"], D)) * 0.05).astype(np.float32)
    w["lnf_w"] = (1.0 + rng.standard_normal(D) * 0.05).astype(np.float32)
    w["lnf_b"] = small(D)
    return w


def encoder_states(cfg: dict, n_clips: int, seed: int = 7) -> np.ndarray:
    """Stand-in encoder outputs [n_clips, Tenc, D]: unit-variance rows like a final-LayerNorm output."""
    rng = np.random.default_rng(seed)
    return rng.standard_normal((n_clips, cfg["Tenc"], cfg["D"]), dtype=np.float32)


def synth_audio(n_windows: int, samples: int = 240000, sr: int = 16000, seed: int = 3) -> np.ndarray:
    """Pink noise (white noise shaped by 1/sqrt(f), unit RMS) x amp~U(0.05,0.5) plus 1-4 tones of
    100-4000 Hz, amp~U(0.05,0.5).  [n_windows, samples] f32."""
    rng = np.random.default_rng(seed)
    out = np.empty((n_windows, samples), np.float32)
    f = np.fft.rfftfreq(samples, 1.0 / sr)
    shape = np.ones_like(f)
    shape[1:] = 1.0 / np.sqrt(f[1:])
    t = np.arange(samples) / sr
    for i in range(n_windows):
        x = np.fft.irfft(np.fft.rfft(rng.standard_normal(samples)) * shape, samples)
        x = x / np.sqrt((x ** 2).mean()) * rng.uniform(0.05, 0.5)
        for _ in range(int(rng.integers(1, 5))):
            x = x + rng.uniform(0.05, 0.5) * np.sin(2 * np.pi * rng.uniform(100, 4000) * t + rng.uniform(0, 2 * np.pi))
        out[i] = x.astype(np.float32)
    return out


def _hz_to_mel(f):
    f = np.asarray(f, np.float64)
    return np.where(f >= 1000.0, 15.0 + np.log(np.maximum(f, 1e-9) / 1000.0) / (math.log(6.4) / 27.0), f / (200.0 / 3))


def _mel_to_hz(m):
    m = np.asarray(m, np.float64)
    return np.where(m >= 15.0, 1000.0 * np.exp((math.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3))


def mel_filterbank(n_mels: int, n_fft: int = 512, sr: int = 16000) -> np.ndarray:
    """Slaney-scale, slaney-normalised triangular filters [n_mels, n_fft/2+1] (nemotron-mel.js:66-110)."""
    n_freq = n_fft // 2 + 1
    freqs = np.linspace(0, sr / 2, n_freq)
    pts = _mel_to_hz(np.linspace(_hz_to_mel(0.0), _hz_to_mel(sr / 2), n_mels + 2))
    fb = np.zeros((n_mels, n_freq))
    for m in range(n_mels):
        lo, c, hi = pts[m], pts[m + 1], pts[m + 2]
        up = (freqs - lo) / (c - lo)
        down = (hi - freqs) / (hi - c)
        fb[m] = np.maximum(0, np.minimum(up, down)) * (2.0 / (hi - lo))
    return fb.astype(np.float32)


def log_mel(audio: np.ndarray, n_mels: int = 128) -> np.ndarray:
    """NeMo front-end with Parakeet settings: preemph 0.97, n_fft 512, Hann 400, hop 160, slaney mels,
    log(mel + 2^-24), per-feature mean/variance normalisation (N-1).  Returns [n_mels, T] f32."""
    x = audio.astype(np.float32)
    x = np.concatenate([x[:1], x[1:] - np.float32(0.97) * x[:-1]]).astype(np.float64)
    x = np.pad(x, 256)
    T = 1 + (x.size - 512) // 160
    win = np.zeros(512)
    win[56:456] = 0.5 - 0.5 * np.cos(2 * np.pi * np.arange(400) / 399)  # symmetric Hann, centred in the frame
    idx = np.arange(512)[None, :] + 160 * np.arange(T)[:, None]
    spec = np.fft.rfft(x[idx] * win, axis=1)
    power = (spec.real ** 2 + spec.imag ** 2).astype(np.float32)
    mel = np.log(power @ mel_filterbank(n_mels).T + np.float32(2.0 ** -24)).T  # [n_mels, T]
    mean = mel.mean(1, keepdims=True)
    std = np.sqrt(((mel - mean) ** 2).sum(1, keepdims=True) / max(1, T - 1))
    return ((mel - mean) / (std + 1e-5)).astype(np.float32)
