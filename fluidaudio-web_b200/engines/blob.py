"""The reference's weight artifact format: one binary blob + a JSON manifest.

Writer: a restatement of scripts/quantize-parakeet-encoder.py:20-59 - matrices [in, out] (linw and the per-layer q, k,
v, pos, out, ff1w1, ff1w2, ff2w1, ff2w2) are quantised to symmetric int8 per OUTPUT COLUMN, convolution weights
(c0w..c4w and the per-layer pw1, pw2, dw; first dimension = output channel) per output channel, everything else stays
f32.  Blob layout: the f32 section first (per-tensor scale vectors and the f32 tensors, in manifest order), then the
int8 section; manifest entries carry ``dims, dtype ("i8" | "f32"), quant ("col" | "grp"), count, scaleCount`` and the
positions ``offset`` / ``scaleOffset`` (in FLOATS) and ``i8ByteOffset`` (in BYTES), as docs/PORTING.md:21-36 describes.

Reader: ``tensor_f32`` is ``raw(k)`` of src/engines/asr-parakeet/raw-encoder.js:56-76 (dequantise one tensor);
``tensor_i8`` hands out the stored int8 values and their scales untouched, for backends that keep them resident.
"""
from __future__ import annotations

import json
import re
from typing import Dict, Tuple

import numpy as np

_MAT_SUFFIX = ("q", "k", "v", "pos", "out", "ff1w1", "ff1w2", "ff2w1", "ff2w2")
_CONV_SUFFIX = ("pw1", "pw2", "dw")


def _is_mat(k: str, dims) -> bool:
    return len(dims) == 2 and (k == "linw" or k.split("_")[-1] in _MAT_SUFFIX)


def _is_conv(k: str) -> bool:
    return bool(re.match(r"^c[0-4]w$", k)) or k.split("_")[-1] in _CONV_SUFFIX


def write_int8_blob(weights: Dict[str, np.ndarray]) -> Tuple[bytes, dict]:
    """f32 tensors (dict order = manifest order) -> (blob, manifest) in the int8 artifact format."""
    f32_blocks, i8_blocks, man = [], [], {}
    for k, arr in weights.items():
        a = np.ascontiguousarray(arr, np.float32)
        dims = list(a.shape)
        if _is_mat(k, dims):
            scale = np.abs(a).max(0) / 127.0
            scale[scale == 0] = 1
            q = np.clip(np.round(a / scale), -127, 127).astype(np.int8)
            man[k] = {"dims": dims, "dtype": "i8", "quant": "col", "count": int(a.size), "scaleCount": dims[1]}
            i8_blocks.append((k, q.reshape(-1)))
            f32_blocks.append(("__scale__" + k, scale.astype(np.float32)))
        elif _is_conv(k):
            cout = dims[0]
            a2 = a.reshape(cout, -1)
            scale = np.abs(a2).max(1) / 127.0
            scale[scale == 0] = 1
            q = np.clip(np.round(a2 / scale[:, None]), -127, 127).astype(np.int8)
            man[k] = {"dims": dims, "dtype": "i8", "quant": "grp", "count": int(a.size), "scaleCount": cout}
            i8_blocks.append((k, q.reshape(-1)))
            f32_blocks.append(("__scale__" + k, scale.astype(np.float32)))
        else:
            man[k] = {"dims": dims, "dtype": "f32", "count": int(a.size)}
            f32_blocks.append((k, a.reshape(-1)))
    blob = bytearray()
    for key, arr in f32_blocks:  # all f32 first (4-byte aligned by construction), then all int8
        off = len(blob) // 4
        if key.startswith("__scale__"):
            man[key[9:]]["scaleOffset"] = off
        else:
            man[key]["offset"] = off
        blob += np.ascontiguousarray(arr, np.float32).tobytes()
    for key, arr in i8_blocks:
        man[key]["i8ByteOffset"] = len(blob)
        blob += np.ascontiguousarray(arr, np.int8).tobytes()
    return bytes(blob), man


def save(path_bin: str, path_manifest: str, blob: bytes, man: dict) -> None:
    with open(path_bin, "wb") as f:
        f.write(blob)
    with open(path_manifest, "w") as f:
        json.dump(man, f)


def load(path_bin: str, path_manifest: str) -> Tuple[bytes, dict]:
    with open(path_bin, "rb") as f:
        blob = f.read()
    with open(path_manifest) as f:
        return blob, json.load(f)


class Blob:
    """Views over one artifact (raw-encoder.js:44-50: the same buffer seen as f32 and as int8)."""

    def __init__(self, blob: bytes, man: dict):
        self.man = man
        self.u8 = np.frombuffer(blob, np.uint8)
        self.f32 = np.frombuffer(blob, np.float32, count=len(blob) // 4)
        self.i8 = self.u8.view(np.int8)

    def is_i8(self, k: str) -> bool:
        return self.man[k].get("dtype") == "i8"

    def tensor_i8(self, k: str):
        """(int8 values in the tensor's dims, f32 scales, quant kind) as stored."""
        m = self.man[k]
        q = self.i8[m["i8ByteOffset"]:m["i8ByteOffset"] + m["count"]].reshape(m["dims"])
        sc = self.f32[m["scaleOffset"]:m["scaleOffset"] + m["scaleCount"]]
        return q, sc, m["quant"]

    def tensor_f32(self, k: str) -> np.ndarray:
        """raw(k): the tensor as f32, dequantised when it is stored int8 (q * scale of its column / output channel)."""
        m = self.man[k]
        if m.get("dtype") != "i8":
            return np.array(self.f32[m["offset"]:m["offset"] + m["count"]]).reshape(m["dims"])
        q, sc, kind = self.tensor_i8(k)
        if kind == "col":
            return (q.astype(np.float32) * sc[None, :]).astype(np.float32)
        q2 = q.reshape(m["dims"][0], -1).astype(np.float32)
        return (q2 * sc[:, None]).astype(np.float32).reshape(m["dims"])

    def as_f32_dict(self) -> Dict[str, np.ndarray]:
        return {k: self.tensor_f32(k) for k in self.man}
