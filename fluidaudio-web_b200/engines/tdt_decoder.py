"""Parakeet TDT decoder (prediction network + joint), host side: loader and batched greedy decode.

Mirrors src/engines/asr-parakeet/raw-decoder-wasm.js: loadWasmDecoder (:12-53: weights by manifest key, the joint's
out matrix quantised to int8 rows with per-row scales) and wasmDecodeProj (:58-70: ids + emission frames for one
window of pre-projected frames).  The device side (fa_tdt_*) decodes all windows of a batch in lock-step; its
arithmetic follows rust/parakeet-decoder/src/lib.rs.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Tuple

import numpy as np

HID, ENC_D, VOCAB, LOGITS, BLANK = 640, 1024, 8193, 8198, 8192
KEYS = ["embed", "l0_W", "l0_R", "l0_B", "l1_W", "l1_R", "l1_B", "encW", "encB", "predW", "predB", "outW", "outB"]


def quantize_out_rows(out_w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """raw-decoder-wasm.js:30-44: per-row symmetric int8 of outW [640, 8198], computed in doubles; Math.round rounds
    halves towards +infinity; an all-zero row gets scale 1; the scale is kept as f32."""
    ow = np.asarray(out_w, np.float32).reshape(HID, -1).astype(np.float64)
    mx = np.abs(ow).max(axis=1)
    sc = np.where(mx / 127 == 0, 1.0, mx / 127)
    q = np.clip(np.floor(ow / sc[:, None] + 0.5), -127, 127).astype(np.int8)
    return q, sc.astype(np.float32)


class TdtDecoder:
    """loadWasmDecoder's result on the CUDA backend: weights resident on the device, one handle."""

    def __init__(self, ctx, weights: Dict[str, np.ndarray], int8: bool = True):
        self.ctx = ctx
        w = {k: np.ascontiguousarray(weights[k], np.float32).reshape(-1) for k in KEYS}
        f = lambda a: a.ctypes.data_as(C.c_void_p)
        self.projW = ctx.uploadF16(w["encW"].reshape(ENC_D, HID), ENC_D, HID)  # the encoder's joint projection (pipeline.js:57-61)
        self.projB = ctx.upload(w["encB"], 1, HID)
        q = sc = None
        if int8:
            q, sc = quantize_out_rows(w["outW"])
            q = np.ascontiguousarray(q)
        h = C.c_void_p()
        ctx._check(ctx._lib.fa_tdt_create(ctx._h, f(w["embed"]), f(w["l0_W"]), f(w["l0_R"]), f(w["l0_B"]), f(w["l1_W"]),
                                          f(w["l1_R"]), f(w["l1_B"]), f(w["predW"]), f(w["predB"]),
                                          None if int8 else f(w["outW"]), f(w["outB"]), f(q) if int8 else None,
                                          f(sc) if int8 else None, C.byref(h)))
        self.h = h
        self.rounds = 0

    def decode_proj(self, proj, W: int, T: int) -> List[Tuple[np.ndarray, np.ndarray]]:
        """proj: device tensor [W*T, 640] of pre-projected frames -> per window (token ids, emission frames)."""
        cap = T * 10  # MAX_SYMBOLS tokens per frame in the worst case (raw-decoder-wasm.js:64-66)
        ids = np.empty(W * cap, np.int32)
        fr = np.empty(W * cap, np.int32)
        cnt = np.empty(W, np.int32)
        rounds = C.c_int()
        p = lambda a: a.ctypes.data_as(C.c_void_p)
        self.ctx._check(self.ctx._lib.fa_tdt_decode_proj(self.ctx._h, self.h, proj.h, W, T, cap, p(ids), p(fr), p(cnt), C.byref(rounds)))
        self.rounds = rounds.value
        return [(ids[w * cap:w * cap + cnt[w]].copy(), fr[w * cap:w * cap + cnt[w]].copy()) for w in range(W)]

    def project(self, frames):
        """The joint's encoder projection riding the encoder's batch (pipeline.js:57-61): [W*T, 1024] -> [W*T, 640]."""
        return self.ctx.matmul(frames, self.projW, dict(bias=self.projB))

    def free(self):
        if self.h:
            self.ctx._check(self.ctx._lib.fa_tdt_free(self.ctx._h, self.h))
            self.h = None
        self.ctx.freeTensor(self.projW)
        self.ctx.freeTensor(self.projB)


def synth_tdt_weights(seed: int = 5, blank_bias: float = 2.0) -> Dict[str, np.ndarray]:
    """Seeded random-init decoder weights in the reference manifest's names and shapes: matrices ~ N(0, 1/fan_in),
    small biases, and a positive bias on the blank logit so that, as with a trained model, most frames emit nothing."""
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
