"""Python face of oracle/parakeet_decoder_port.c (the reference's TDT decoder restated in C).

TEST INFRASTRUCTURE ONLY.  ``TdtOracle`` takes the weight dictionary of the reference's decoder manifest
(keys of src/engines/asr-parakeet/raw-decoder-wasm.js:26) and offers ``decode`` / ``decode_proj`` with the
meaning of ``wasmDecode`` / ``wasmDecodeProj`` (:58-81), plus a batch form that decodes independent
windows on several host threads (one private state block per thread).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build_oracle
from .ref_wasm import TDT_KEYS, quantize_out_rows

HID, ENC_D, VOCAB, LOGITS, BLANK = 640, 1024, 8193, 8198, 8192

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
_lib = C.CDLL(build_oracle.build())
_lib.tdt_create.restype = C.c_void_p
_lib.tdt_create.argtypes = [_f32p] * 13
_lib.tdt_set_out_q.argtypes = [C.c_void_p, C.POINTER(C.c_int8), _f32p]
_lib.tdt_set_out_q.restype = None
_lib.tdt_destroy.argtypes = [C.c_void_p]
_lib.tdt_destroy.restype = None
for _n in ("tdt_decode", "tdt_decode_proj"):
    getattr(_lib, _n).argtypes = [C.c_void_p, _f32p, C.c_uint32, _i32p, _i32p]
    getattr(_lib, _n).restype = C.c_int32
_lib.tdt_joint_logits.argtypes = [C.c_void_p, C.c_int32, _f32p, _f32p]
_lib.tdt_joint_logits.restype = None
_lib.tdt_last_logits.argtypes = [C.c_void_p, _f32p]
_lib.tdt_last_logits.restype = None
_lib.tdt_decode_proj_batch.argtypes = [C.POINTER(C.c_void_p), C.c_int, _f32p, C.c_uint32, C.c_int32, C.c_int32,
                                       _i32p, _i32p, _i32p]
_lib.tdt_decode_proj_batch.restype = None


def _fp(a):
    return a.ctypes.data_as(_f32p)


class TdtOracle:
    def __init__(self, weights: dict, int8: bool = True, threads: int = 1):
        self.w = {k: np.ascontiguousarray(weights[k], np.float32).reshape(-1) for k in TDT_KEYS}
        self.q = self.scale = None
        if int8:
            self.q, self.scale = quantize_out_rows(self.w["outW"].reshape(HID, LOGITS))
            self.q = np.ascontiguousarray(self.q)
        self.threads = max(1, int(threads))
        self._hs = []
        for _ in range(self.threads):
            h = _lib.tdt_create(*[_fp(self.w[k]) for k in TDT_KEYS])
            if self.q is not None:
                _lib.tdt_set_out_q(h, self.q.ctypes.data_as(C.POINTER(C.c_int8)), _fp(self.scale))
            self._hs.append(h)

    def __del__(self):
        for h in getattr(self, "_hs", []):
            _lib.tdt_destroy(h)
        self._hs = []

    def _run(self, fn, frames, tenc):
        frames = np.ascontiguousarray(frames, np.float32).reshape(-1)
        ids = np.empty(tenc * 10, np.int32)
        fr = np.empty(tenc * 10, np.int32)
        n = fn(self._hs[0], _fp(frames), tenc, ids.ctypes.data_as(_i32p), fr.ctypes.data_as(_i32p))
        return ids[:n].copy(), fr[:n].copy()

    def decode(self, frames, tenc):
        return self._run(_lib.tdt_decode, frames, tenc)

    def decode_proj(self, proj, tenc):
        return self._run(_lib.tdt_decode_proj, proj, tenc)

    def joint_logits(self, token, proj):
        out = np.empty(LOGITS, np.float32)
        _lib.tdt_joint_logits(self._hs[0], int(token), _fp(np.ascontiguousarray(proj, np.float32)), _fp(out))
        return out

    def last_logits(self):
        """Logits of the last joint step the previous decode call evaluated."""
        out = np.empty(LOGITS, np.float32)
        _lib.tdt_last_logits(self._hs[0], _fp(out))
        return out

    def decode_proj_batch(self, proj, nwin, tenc):
        """proj [nwin, tenc, 640] -> list of (ids, frames) per window."""
        proj = np.ascontiguousarray(proj, np.float32).reshape(-1)
        cap = tenc * 10
        ids = np.empty(nwin * cap, np.int32)
        fr = np.empty(nwin * cap, np.int32)
        cnt = np.empty(nwin, np.int32)
        hs = (C.c_void_p * self.threads)(*self._hs)
        _lib.tdt_decode_proj_batch(hs, self.threads, _fp(proj), tenc, nwin, cap, ids.ctypes.data_as(_i32p),
                                   fr.ctypes.data_as(_i32p), cnt.ctypes.data_as(_i32p))
        return [(ids[w * cap:w * cap + cnt[w]].copy(), fr[w * cap:w * cap + cnt[w]].copy()) for w in range(nwin)]


def synth_tdt_weights(seed: int = 5, blank_bias: float = 2.0) -> dict:
    """Seeded random-init decoder weights in the reference manifest's names and shapes.

    Matrices ~ N(0, 1/fan_in); LSTM biases small; the blank logit gets a positive bias so that, as with a
    trained model, most frames emit nothing and a fraction emit one or more tokens.
    """
    rng = np.random.default_rng(seed)

    def mat(*shape, fan_in):
        return (rng.standard_normal(shape) / np.sqrt(fan_in)).astype(np.float32)

    w = {"embed": mat(VOCAB, HID, fan_in=1.0)}
    for l in (0, 1):
        w[f"l{l}_W"] = mat(4 * HID, HID, fan_in=HID)
        w[f"l{l}_R"] = mat(4 * HID, HID, fan_in=HID)
        w[f"l{l}_B"] = (0.1 * rng.standard_normal(8 * HID)).astype(np.float32)
    w["encW"] = mat(ENC_D, HID, fan_in=ENC_D)
    w["encB"] = (0.1 * rng.standard_normal(HID)).astype(np.float32)
    w["predW"] = mat(HID, HID, fan_in=HID)
    w["predB"] = (0.1 * rng.standard_normal(HID)).astype(np.float32)
    w["outW"] = mat(HID, LOGITS, fan_in=HID)
    ob = (0.1 * rng.standard_normal(LOGITS)).astype(np.float32)
    ob[BLANK] += blank_bias
    w["outB"] = ob
    return w
