"""Python face of oracle/nemo_mel_port.c (the reference's JsPreprocessor / ParakeetMel restated in C).

TEST INFRASTRUCTURE ONLY.  ``parakeet_mel(audio)`` has the meaning of ``ParakeetMel.process``
(src/engines/asr-parakeet/parakeet-mel.js:16-21): features [nMels, length] with length = floor(N/160),
log guard 2^-24, per-feature normalisation; ``nemotron_mel`` is ``JsPreprocessor.process`` (guard 1e-10, raw log-mel
over N/160 + 1 frames, src/engines/asr-nemotron/nemotron-mel.js:428-441).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build_oracle

_lib = C.CDLL(build_oracle.build())
_f32p = C.POINTER(C.c_float)
_lib.mel_compute_raw.argtypes = [_f32p, C.c_int, C.c_int, C.c_double, _f32p, C.POINTER(C.c_int)]
_lib.mel_compute_raw.restype = C.c_int
_lib.mel_normalize.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _f32p]
_lib.mel_normalize.restype = None
_lib.mel_filterbank.argtypes = [C.c_int, _f32p, C.POINTER(C.c_int32)]
_lib.mel_filterbank.restype = None


def raw_mel(audio: np.ndarray, n_mels: int = 128, log_guard: float = 2.0 ** -24):
    a = np.ascontiguousarray(audio, np.float32).reshape(-1)
    n_frames = a.size // 160 + 1 if a.size else 0
    raw = np.zeros((n_mels, max(n_frames, 1)), np.float32)
    nf = C.c_int()
    feat = _lib.mel_compute_raw(a.ctypes.data_as(_f32p), a.size, n_mels, log_guard, raw.ctypes.data_as(_f32p), C.byref(nf))
    return raw[:, :nf.value] if nf.value else raw[:, :0], feat


def parakeet_mel(audio: np.ndarray, n_mels: int = 128) -> np.ndarray:
    raw, feat = raw_mel(audio, n_mels, 2.0 ** -24)
    if feat == 0:
        return np.zeros((n_mels, 0), np.float32)
    raw = np.ascontiguousarray(raw)
    out = np.empty((n_mels, feat), np.float32)
    _lib.mel_normalize(raw.ctypes.data_as(_f32p), n_mels, raw.shape[1], feat, out.ctypes.data_as(_f32p))
    return out


def nemotron_mel(audio: np.ndarray, n_mels: int = 128) -> np.ndarray:
    return raw_mel(audio, n_mels, 1e-10)[0]


def filterbank(n_mels: int = 128):
    fb = np.empty((n_mels, 257), np.float32)
    bounds = np.empty((n_mels, 2), np.int32)
    _lib.mel_filterbank(n_mels, fb.ctypes.data_as(_f32p), bounds.ctypes.data_as(C.POINTER(C.c_int32)))
    return fb, bounds
