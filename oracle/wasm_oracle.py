"""Python face of the CPU oracle: the reference's WasmContext, method for method.

TEST INFRASTRUCTURE ONLY.  Only tests/, __graft_entry__.smoke() and bench.py's CPU
baseline legs may import this module; the product package never does.

Every method has the name, argument meaning and return shape of the reference's CPU
backend class (src/gpu/wasm-context.js:46-777) so parity tests read like the
reference's own cross-backend gate (scripts/backend-conformance.mjs).  The arithmetic
lives in oracle/wasm_kernels_port.c; this file only stages arrays the way the JS does
(which copies are made, what is sliced out, epilogue order).
"""
from __future__ import annotations

import ctypes as C
import math
import os

import numpy as np

from . import build_oracle

ACT = {"none": 0, "gelu": 1, "tanh": 2, "relu": 3, "silu": 4, "gelu_erf": 5}  # src/gpu/kernels/actf.js:24

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_i32p = C.POINTER(C.c_int32)
_sz = C.c_size_t


def _load() -> C.CDLL:
    lib = C.CDLL(build_oracle.build())
    sigs = {
        "wk_matmul_f32": [_f32p, _f32p, _f32p, _sz, _sz, _sz],
        "wk_matmul_f32_mt": [_f32p, _f32p, _f32p, _sz, _sz, _sz],
        "wk_conv1d_f32": [_f32p, _f32p, _f32p] + [_sz] * 9,
        "wk_matmul_int8": [_f32p, _u8p, _f32p, _f32p, _sz, _sz, _sz],
        "wk_matmul_int8_kj": [_f32p, _u8p, _f32p, _f32p, _sz, _sz, _sz],
        "wk_matmul_int8_mt": [_f32p, _u8p, _f32p, _f32p, _sz, _sz, _sz],
        "wk_matmul_nbits": [_f32p, _u8p, _f32p, _u8p, _f32p] + [_sz] * 6,
        "wk_matmul_nbits_mt": [_f32p, _u8p, _f32p, _u8p, _f32p] + [_sz] * 6,
        "js_bias_act_columns": [_f32p, _sz, _sz, _f32p, C.c_int],
        "js_bias_act_rows": [_f32p, _sz, _sz, _f32p, C.c_int],
        "js_residual_add": [_f32p, _f32p, _sz],
        "js_layernorm": [_f32p, _f32p, _f32p, _f32p, _sz, _sz, C.c_double],
        "js_softmax": [_f32p, _f32p, _sz, _sz],
        "js_ewise": [_f32p, _f32p, _f32p, _sz, _sz, C.c_int, C.c_int],
        "js_scale": [_f32p, _f32p, _sz, C.c_double],
        "js_silu_op": [_f32p, _f32p, _sz],
        "js_relu_op": [_f32p, _f32p, _sz],
        "js_glu": [_f32p, _f32p, _sz, _sz],
        "js_transpose": [_f32p, _f32p, _sz, _sz],
        "js_slice_cols": [_f32p, _f32p, _sz, _sz, _sz, _sz],
        "js_set_cols": [_f32p, _sz, _f32p, _sz, _sz, _sz],
        "js_bmm_qk": [_f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, _sz, C.c_int],
        "js_bmm_pv": [_f32p, _f32p, _f32p, _sz, _sz, _sz, _sz, _sz],
        "js_rel_shift_b": [_f32p, _f32p, _sz, _sz],
        "js_sub_reshape": [_f32p, _f32p, _sz, _sz, _sz],
        "js_conv2d": [_f32p, _f32p, _f32p, _f32p] + [_sz] * 8 + [C.c_long] * 4 + [_sz, C.c_int],
        "int8_gemm_i32": [_i8p, _u8p, _i32p, _sz, _sz, _sz],
        "mulberry32_fill_f32": [C.POINTER(C.c_uint32), _f32p, _sz],
        "mulberry32_fill_u8": [C.POINTER(C.c_uint32), _u8p, _sz],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = None
    lib.js_apply_act.argtypes = [C.c_double, C.c_int]
    lib.js_apply_act.restype = C.c_double
    lib.oracle_num_threads.restype = C.c_int
    lib.oracle_set_num_threads.argtypes = [C.c_int]
    lib.oracle_set_num_threads.restype = None
    return lib


LIB = _load()


def _f(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_f32p)


def _b(a: np.ndarray):
    assert a.dtype == np.uint8 and a.flags.c_contiguous
    return a.ctypes.data_as(_u8p)


class T:
    """CPU tensor {data, rows, cols} (wasm-context.js:7)."""

    __slots__ = ("data", "rows", "cols")

    def __init__(self, data: np.ndarray, rows: int, cols: int):
        self.data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        assert self.data.size >= rows * cols
        self.rows, self.cols = rows, cols

    def array(self) -> np.ndarray:
        return self.data[: self.rows * self.cols].reshape(self.rows, self.cols)


class Bytes:
    """Packed byte payload {bytes} (wasm-context.js:59-62)."""

    __slots__ = ("bytes",)

    def __init__(self, b: np.ndarray):
        self.bytes = np.ascontiguousarray(b).view(np.uint8).reshape(-1).copy()


class Mulberry32:
    """Seeded generator of scripts/backend-conformance.mjs:46-54."""

    def __init__(self, seed: int = 0x5EED):
        self._s = C.c_uint32(seed & 0xFFFFFFFF)

    def data(self, n: int) -> np.ndarray:  # mkData: rand() - 0.5 as f32
        out = np.empty(n, np.float32)
        LIB.mulberry32_fill_f32(C.byref(self._s), _f(out), n)
        return out

    def bytes(self, n: int) -> np.ndarray:  # mkBytes: floor(rand()*256)
        out = np.empty(n, np.uint8)
        LIB.mulberry32_fill_u8(C.byref(self._s), _b(out), n)
        return out


class WasmOracle:
    """Method-for-method mirror of WasmContext (src/gpu/wasm-context.js:46)."""

    backend = "wasm"

    def __init__(self, threads: bool = False):
        # threads=True uses the bit-identical multi-threaded forms of the three GEMMs
        # (rows/columns are independent); default follows the reference's serial loops.
        # For int8 that is the i,k,j loop order: every output still sums its k terms in order, so the
        # result is bit-identical to the reference's i,j,k order while the weight bytes are read row-wise.
        self._mt = threads
        self._int8_order = "ikj" if threads else "ijk"

    # -- memory / tensors (:53-123) ------------------------------------------------
    def upload(self, data, rows, cols):
        return T(np.array(data, dtype=np.float32, copy=True), rows, cols)

    uploadF16 = upload  # :64-66, f16 is a storage optimisation the CPU twin ignores

    def alloc(self, rows, cols):
        return T(np.zeros(rows * cols, np.float32), rows, cols)

    allocF16 = alloc

    def uploadBytes(self, typed):
        return Bytes(np.asarray(typed))

    def download(self, t):
        return t.data[: t.rows * t.cols].copy()

    downloadF16 = download

    def stageDownload(self, t):  # :141, StagedRead.read :44 (single use)
        data = t.data[: t.rows * t.cols].copy()

        class _Staged:
            def read(self_inner):
                return data

        return _Staged()

    def rowsView(self, t, rows):
        v = T.__new__(T)
        v.data, v.rows, v.cols = t.data[: rows * t.cols], rows, t.cols
        return v

    def reshapeView(self, t, rows, cols):
        v = T.__new__(T)
        v.data, v.rows, v.cols = t.data[: rows * cols], rows, cols
        return v

    def ensureTensor(self, t):
        return t if isinstance(t, T) else self.upload(t["data"], t["rows"], t["cols"])

    # arenas / batching are GPU-pool concepts: inert on the CPU twin (:104-123)
    def destroy(self):
        pass

    def beginBatch(self):
        pass

    def endBatch(self):
        pass

    def withBatchSync(self, fn):
        return fn()

    withBatch = withBatchSync

    def pushArena(self):
        return []

    def popArena(self, handle=None):
        pass

    def trimPool(self, budget=0):
        pass

    def pin(self, t, toParent=False):
        return t

    def freeTensor(self, t):
        pass

    # -- hot kernels (:135-213) ----------------------------------------------------
    def matmul(self, a, b, opts=None, bias=None, act="none", add=None):
        if opts:
            bias, act, add = opts.get("bias", bias), opts.get("act", act) or "none", opts.get("add", add)
        M, K, N = a.rows, a.cols, b.cols
        assert b.rows == K
        out = np.empty(M * N, np.float32)
        fn = LIB.wk_matmul_f32_mt if self._mt else LIB.wk_matmul_f32
        fn(_f(a.data), _f(b.data), _f(out), M, K, N)
        LIB.js_bias_act_columns(_f(out), M, N, _f(bias.data) if bias is not None else None, ACT[act])
        if add is not None:
            LIB.js_residual_add(_f(out), _f(add.data), M * N)
        return T(out, M, N)

    def matmulV2(self, a, b, opts=None, bias=None, act="none"):
        return self.matmul(a, b, opts, bias=bias, act=act)

    matmulV3 = matmulV4 = matmulF16 = matmulV2

    def matmulInt8(self, a, wq, scale, N, K, bias=None, act="none", loop_order=None):
        loop_order = loop_order or self._int8_order
        M = a.rows
        assert a.cols == K and wq.bytes.size >= K * N
        out = np.empty(M * N, np.float32)
        fn = {"ijk": LIB.wk_matmul_int8_mt if self._mt else LIB.wk_matmul_int8, "ikj": LIB.wk_matmul_int8_kj}[loop_order]
        fn(_f(a.data), _b(wq.bytes), _f(scale.data), _f(out), M, N, K)
        LIB.js_bias_act_columns(_f(out), M, N, _f(bias.data) if bias is not None else None, ACT[act])
        return T(out, M, N)

    def matmulNBits(self, a, bq, scales, zp, N, blockSize=32):
        M, K = a.rows, a.cols
        nblk = math.ceil(K / blockSize)
        zpb = math.ceil(nblk / 2)
        out = np.empty(M * N, np.float32)
        fn = LIB.wk_matmul_nbits_mt if self._mt else LIB.wk_matmul_nbits
        fn(_f(a.data), _b(bq.bytes), _f(scales.data), _b(zp.bytes), _f(out), M, N, K, nblk, zpb, blockSize)
        return T(out, M, N)

    # -- conv (:220-264 grouped path, :632-685) --------------------------------------
    def conv1d(self, x, w, opts=None, cout=None, k=None, bias=None, stride=1, pad=0, padLeft=None, padRight=None,
               dilation=1, groups=1, act="none"):
        if opts:
            cout, k, bias = opts.get("cout", cout), opts.get("k", k), opts.get("bias", bias)
            stride, pad, dilation = opts.get("stride", stride), opts.get("pad", pad), opts.get("dilation", dilation)
            padLeft, padRight = opts.get("padLeft", padLeft), opts.get("padRight", padRight)
            groups, act = opts.get("groups", groups), opts.get("act", act) or "none"
        padLeft = pad if padLeft is None else padLeft
        padRight = pad if padRight is None else padRight
        Cin, L = x.rows, x.cols
        Lout = (L + padLeft + padRight - dilation * (k - 1) - 1) // stride + 1
        if groups == 1:
            # im2col (zero-filled) then the f32 GEMM, :226-250
            cols = np.zeros((Cin * k, Lout), np.float32)
            xa = x.array()
            for ci in range(Cin):
                for kk in range(k):
                    off = kk * dilation - padLeft
                    lo = np.arange(Lout)
                    li = lo * stride + off
                    ok = (li >= 0) & (li < L)
                    cols[ci * k + kk, lo[ok]] = xa[ci, li[ok]]
            out = self.matmul(T(w.data, cout, Cin * k), T(cols, Cin * k, Lout))
            LIB.js_bias_act_rows(_f(out.data), cout, Lout, _f(bias.data) if bias is not None else None, ACT[act])
            return out
        out = np.empty(cout * Lout, np.float32)
        LIB.wk_conv1d_f32(_f(x.data), _f(w.data), _f(out), cout, Cin, L, Lout, k, stride, padLeft, dilation, groups)
        LIB.js_bias_act_rows(_f(out), cout, Lout, _f(bias.data) if bias is not None else None, ACT[act])
        return T(out, cout, Lout)

    def conv2d(self, x, w, opts=None, cin=None, h=None, w_=None, kh=None, kw=None, bias=None, strideH=1, strideW=1,
               padH=0, padW=0, padTop=None, padBottom=None, padLeft=None, padRight=None, groups=1, act="none", cout=None):
        if isinstance(opts, dict):  # JS-style options object (:632-654)
            o = opts
            cout, cin, h, w_, kh, kw = o["cout"], o["cin"], o["h"], o["w"], o["kh"], o["kw"]
            bias, strideH, strideW = o.get("bias"), o.get("strideH", 1), o.get("strideW", 1)
            padH, padW = o.get("padH", 0), o.get("padW", 0)
            padTop, padBottom, padLeft, padRight = o.get("padTop"), o.get("padBottom"), o.get("padLeft"), o.get("padRight")
            groups, act = o.get("groups", 1), o.get("act", "none") or "none"
        elif opts is not None:
            cout = opts  # positional form: conv2d(x, w, cout, cin, h, w, kh, kw, ...)
        padTop = padH if padTop is None else padTop
        padBottom = padH if padBottom is None else padBottom
        padLeft = padW if padLeft is None else padLeft
        padRight = padW if padRight is None else padRight
        Ho = (h + padTop + padBottom - kh) // strideH + 1
        Wo = (w_ + padLeft + padRight - kw) // strideW + 1
        out = np.empty(cout * Ho * Wo, np.float32)
        LIB.js_conv2d(_f(x.data), _f(w.data), _f(bias.data) if bias is not None else None, _f(out), cout, cin, h, w_,
                      kh, kw, strideH, strideW, padTop, padBottom, padLeft, padRight, groups, ACT[act])
        return T(out, cout, Ho * Wo)

    # -- cheap kernels (:308-563) ----------------------------------------------------
    def layernorm(self, x, gamma, beta, eps=1e-5):
        out = np.empty(x.rows * x.cols, np.float32)
        LIB.js_layernorm(_f(x.data), _f(gamma.data), _f(beta.data), _f(out), x.rows, x.cols, eps)
        return T(out, x.rows, x.cols)

    def softmax(self, x):
        out = np.empty(x.rows * x.cols, np.float32)
        LIB.js_softmax(_f(x.data), _f(out), x.rows, x.cols)
        return T(out, x.rows, x.cols)

    def ewise(self, a, b, op):
        out = np.empty(a.rows * a.cols, np.float32)
        LIB.js_ewise(_f(a.data), _f(b.data), _f(out), a.rows, a.cols, int(b.rows == 1), 1 if op == "mul" else 0)
        return T(out, a.rows, a.cols)

    def add(self, a, b):
        return self.ewise(a, b, "add")

    def mul(self, a, b):
        return self.ewise(a, b, "mul")

    def scale(self, x, s):
        out = np.empty(x.rows * x.cols, np.float32)
        LIB.js_scale(_f(x.data), _f(out), out.size, float(s))
        return T(out, x.rows, x.cols)

    def silu(self, x):
        out = np.empty(x.rows * x.cols, np.float32)
        LIB.js_silu_op(_f(x.data), _f(out), out.size)
        return T(out, x.rows, x.cols)

    def relu(self, x):
        out = np.empty(x.rows * x.cols, np.float32)
        LIB.js_relu_op(_f(x.data), _f(out), out.size)
        return T(out, x.rows, x.cols)

    def glu(self, x):
        Cc, Tt = x.rows // 2, x.cols
        out = np.empty(Cc * Tt, np.float32)
        LIB.js_glu(_f(x.data), _f(out), Cc, Tt)
        return T(out, Cc, Tt)

    def transpose(self, x):
        out = np.empty(x.rows * x.cols, np.float32)
        LIB.js_transpose(_f(x.data), _f(out), x.rows, x.cols)
        return T(out, x.cols, x.rows)

    def sliceCols(self, x, col0, width):
        out = np.empty(x.rows * width, np.float32)
        LIB.js_slice_cols(_f(x.data), _f(out), x.rows, x.cols, col0, width)
        return T(out, x.rows, width)

    def setCols(self, dst, src, col0):
        LIB.js_set_cols(_f(dst.data), dst.cols, _f(src.data), src.rows, src.cols, col0)
        return dst

    def sliceRows(self, x, row0, count):
        return T(x.data[row0 * x.cols:(row0 + count) * x.cols].copy(), count, x.cols)

    def copyRows(self, dst, src, rowOffset):
        n = src.rows * src.cols
        dst.data[rowOffset * dst.cols: rowOffset * dst.cols + n] = src.data[:n]
        return dst

    def concatRows(self, tensors):
        cols = tensors[0].cols
        rows = sum(t.rows for t in tensors)
        return T(np.concatenate([t.data[: t.rows * t.cols] for t in tensors]), rows, cols)

    def bmmQK(self, q, b, qb, H, HD, W=1, bShared=False):
        Tq = q.rows // W
        Tb = b.rows if bShared else b.rows // W
        out = np.empty(W * H * Tq * Tb, np.float32)
        LIB.js_bmm_qk(_f(q.data), _f(b.data), _f(qb.data) if qb is not None else None, _f(out), q.rows, b.rows, H, HD,
                      W, int(bShared))
        return T(out, W * H * Tq, Tb)

    def bmmPV(self, p, v, H, HD, W=1):
        Tq = p.rows // (W * H)
        out = np.empty(W * Tq * H * HD, np.float32)
        LIB.js_bmm_pv(_f(p.data), _f(v.data), _f(out), p.rows, v.rows, H, HD, W)
        return T(out, W * Tq, H * HD)

    def relShiftB(self, x, H):
        t = x.rows // H
        out = np.empty(H * t * t, np.float32)
        LIB.js_rel_shift_b(_f(x.data), _f(out), x.rows, H)
        return T(out, H * t, t)

    def relShift(self, x):
        return self.relShiftB(x, 1)

    def subReshape(self, x, Cc, Tsub, F):
        out = np.empty(Tsub * Cc * F, np.float32)
        LIB.js_sub_reshape(_f(x.data), _f(out), Cc, Tsub, F)
        return T(out, Tsub, Cc * F)


def int8_gemm_i32(aq: np.ndarray, wq_kn: np.ndarray) -> np.ndarray:
    """Exact int32 accumulators of int8 activations [M,K] x int8 weights in [K][N] byte order."""
    M, K = aq.shape
    N = wq_kn.size // K
    acc = np.empty((M, N), np.int32)
    LIB.int8_gemm_i32(np.ascontiguousarray(aq, np.int8).ctypes.data_as(_i8p), _b(np.ascontiguousarray(wq_kn).view(np.uint8).reshape(-1)),
                      acc.ctypes.data_as(_i32p), M, N, K)
    return acc
