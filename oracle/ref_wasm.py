"""Drives the reference's own compiled kernels (the shipped .wasm files) through oracle/wasm_exec.py.

TEST INFRASTRUCTURE ONLY.  These classes stage inputs the way the reference's JS hosts do and call the
module's exports, so their outputs are outputs of the reference itself:

* ``RefWasmKernels``  — ``src/gpu/wasm-kernels.wasm`` as ``WasmContext`` calls it
  (``src/gpu/wasm-context.js:135-156`` matmul, ``:171-189`` matmulInt8, ``:192-213`` matmulNBits,
  ``:245-262`` grouped conv1d): ``wasm_reset``, one ``wasm_alloc`` per operand in the same order, copy
  in, call, slice out.  Bias / activation / residual are NOT part of the module (the JS applies them),
  so these methods return the bare accumulations.
* ``RefWasmTdtDecoder`` — ``src/engines/asr-parakeet/parakeet-decoder.wasm`` as
  ``raw-decoder-wasm.js:12-81`` loads and calls it (weights copied once in manifest-key order,
  optional int8 out-matrix with per-row scales, ``decode`` / ``decode_proj``).

The modules are read from a reference checkout; they are never copied into this repository.  Machines
without the checkout use the fixtures under tests/golden/ that tests/golden/gen_wasm_golden.py wrote
from these classes.
"""
from __future__ import annotations

import os

import numpy as np

from .wasm_exec import Instance

KERNELS_WASM = "src/gpu/wasm-kernels.wasm"
DECODER_WASM = "src/engines/asr-parakeet/parakeet-decoder.wasm"


def reference_root():
    """Directory of the reference checkout - $FA_REFERENCE_ROOT, else a `reference` directory beside this repository -
    or None when this machine has none."""
    beside = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
    for cand in (os.environ.get("FA_REFERENCE_ROOT"), beside):
        if cand and os.path.exists(os.path.join(cand, KERNELS_WASM)):
            return cand
    return None


class RefWasmKernels:
    def __init__(self, root: str | None = None):
        root = root or reference_root()
        if root is None:
            raise FileNotFoundError("no reference checkout with " + KERNELS_WASM)
        with open(os.path.join(root, KERNELS_WASM), "rb") as f:
            self.inst = Instance(f.read())

    def _put(self, arr):
        arr = np.ascontiguousarray(arr)
        p = self.inst.call("wasm_alloc", arr.nbytes)
        return p, arr

    def matmul_f32(self, a, b):
        M, K = a.shape
        N = b.shape[1]
        ex = self.inst
        ex.call("wasm_reset")
        ap = ex.call("wasm_alloc", M * K * 4)
        bp = ex.call("wasm_alloc", K * N * 4)
        cp = ex.call("wasm_alloc", M * N * 4)
        ex.write(ap, a.astype(np.float32))
        ex.write(bp, b.astype(np.float32))
        ex.call("matmul_f32", ap, bp, cp, M, K, N)
        return ex.read(cp, M * N, np.float32).reshape(M, N)

    def matmul_int8(self, a, wq_bytes, scale, N, K):
        M = a.shape[0]
        ex = self.inst
        ex.call("wasm_reset")
        ap = ex.call("wasm_alloc", M * K * 4)
        wp = ex.call("wasm_alloc", wq_bytes.size)
        sp = ex.call("wasm_alloc", N * 4)
        yp = ex.call("wasm_alloc", M * N * 4)
        ex.write(ap, a.astype(np.float32))
        ex.write(wp, wq_bytes.view(np.uint8))
        ex.write(sp, scale.astype(np.float32))
        ex.call("matmul_int8", ap, wp, sp, yp, M, N, K)
        return ex.read(yp, M * N, np.float32).reshape(M, N)

    def matmul_nbits(self, a, bq, scales, zp, N, block_size=32):
        M, K = a.shape
        nblk = -(-K // block_size)
        zpb = -(-nblk // 2)
        ex = self.inst
        ex.call("wasm_reset")
        ap = ex.call("wasm_alloc", M * K * 4)
        bqp = ex.call("wasm_alloc", bq.size)
        scp = ex.call("wasm_alloc", scales.size * 4)
        zpp = ex.call("wasm_alloc", zp.size)
        yp = ex.call("wasm_alloc", M * N * 4)
        ex.write(ap, a.astype(np.float32))
        ex.write(bqp, bq.view(np.uint8))
        ex.write(scp, scales.astype(np.float32))
        ex.write(zpp, zp.view(np.uint8))
        ex.call("matmul_nbits", ap, bqp, scp, zpp, yp, M, N, K, nblk, zpb, block_size)
        return ex.read(yp, M * N, np.float32).reshape(M, N)

    def conv1d_f32(self, x, w, cout, k, stride=1, pad_left=0, pad_right=0, dilation=1, groups=1):
        Cin, L = x.shape
        Lout = (L + pad_left + pad_right - dilation * (k - 1) - 1) // stride + 1
        ex = self.inst
        ex.call("wasm_reset")
        xp = ex.call("wasm_alloc", Cin * L * 4)
        wp = ex.call("wasm_alloc", w.size * 4)
        yp = ex.call("wasm_alloc", cout * Lout * 4)
        ex.write(xp, x.astype(np.float32))
        ex.write(wp, w.astype(np.float32))
        ex.call("conv1d_f32", xp, wp, yp, cout, Cin, L, Lout, k, stride, pad_left, dilation, groups)
        return ex.read(yp, cout * Lout, np.float32).reshape(cout, Lout)


TDT_KEYS = ["embed", "l0_W", "l0_R", "l0_B", "l1_W", "l1_R", "l1_B", "encW", "encB", "predW", "predB", "outW", "outB"]


def quantize_out_rows(out_w: np.ndarray):
    """Per-row symmetric int8 of the joint's out matrix, as raw-decoder-wasm.js:30-44 does it in JS doubles.

    ``Math.round`` rounds halves up (toward +inf), unlike rint; ``mx / 127 || 1`` maps an all-zero row to 1.
    The scale is stored in a Float32Array, the division uses the double.
    """
    ow = out_w.astype(np.float64)
    mx = np.abs(ow).max(axis=1)
    sc = np.where(mx / 127 == 0, 1.0, mx / 127)
    q = np.clip(np.floor(ow / sc[:, None] + 0.5), -127, 127).astype(np.int8)
    return q, sc.astype(np.float32)


class RefWasmTdtDecoder:
    def __init__(self, weights: dict, int8: bool = True, root: str | None = None):
        root = root or reference_root()
        if root is None:
            raise FileNotFoundError("no reference checkout with " + DECODER_WASM)
        with open(os.path.join(root, DECODER_WASM), "rb") as f:
            self.inst = ex = Instance(f.read())
        ex.call("reset_to", ex.global_value("__heap_base"))
        ptrs = []
        for k in TDT_KEYS:
            arr = np.ascontiguousarray(weights[k], np.float32).reshape(-1)
            p = ex.call("alloc", arr.nbytes)
            ex.write(p, arr)
            ptrs.append(p)
        ex.call("set_weights", *ptrs)
        if int8:
            q, sc = quantize_out_rows(np.asarray(weights["outW"], np.float32).reshape(640, -1))
            qp = ex.call("alloc", q.nbytes)
            ex.write(qp, q)
            sp = ex.call("alloc", sc.nbytes)
            ex.write(sp, sc)
            ex.call("set_out_q", qp, sp)
        self.mark = ex.call("bump_mark")

    def _decode(self, fn, frames, tenc):
        ex = self.inst
        ex.call("reset_to", self.mark)
        frames = np.ascontiguousarray(frames, np.float32).reshape(-1)
        fp = ex.call("alloc", frames.nbytes)
        ex.write(fp, frames)
        idp = ex.call("alloc", tenc * 10 * 4)
        frp = ex.call("alloc", tenc * 10 * 4)
        n = ex.call(fn, fp, tenc, idp, frp)
        return ex.read(idp, n, np.int32), ex.read(frp, n, np.int32)

    def decode(self, frames, tenc):
        """frames [tenc, 1024] encoder output."""
        return self._decode("decode", frames, tenc)

    def decode_proj(self, proj, tenc):
        """proj [tenc, 640] pre-projected frames (encoder projection and its bias already applied)."""
        return self._decode("decode_proj", proj, tenc)
