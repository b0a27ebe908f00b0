"""CudaContext: the reference's ComputeContext interface on the C-ABI library.

Method names, argument meaning and error behaviour follow src/gpu/compute.d.ts:106-255
(and the two existing implementations, src/gpu/compute.js and src/gpu/wasm-context.js);
options objects become keyword arguments.  Tensors are opaque handles: engine code uses
download / stageDownload / rowsView / ensureTensor, never the storage.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, Optional, Sequence

import numpy as np

from . import _lib

ACT = {"none": 0, "gelu": 1, "tanh": 2, "relu": 3, "silu": 4, "gelu_erf": 5}  # src/gpu/kernels/actf.js:24


class CudaError(RuntimeError):
    """Raised for every non-zero status of the C ABI (the reference throws a JS Error)."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


class Tensor:
    """2-D row-major tensor handle {rows, cols}; storage is backend-owned (compute.d.ts:12-15)."""

    __slots__ = ("h", "rows", "cols", "f16", "view")

    def __init__(self, h: int, rows: int, cols: int, f16: bool = False, view: bool = False):
        self.h, self.rows, self.cols, self.f16, self.view = h, rows, cols, f16, view

    def __repr__(self):
        return f"Tensor({self.rows}x{self.cols}{', f16' if self.f16 else ''}{', view' if self.view else ''})"


class PackedBytes:
    """Opaque packed-weight handle from uploadBytes (compute.d.ts:34)."""

    __slots__ = ("h", "nbytes")

    def __init__(self, h: int, nbytes: int):
        self.h, self.nbytes = h, nbytes


class StagedRead:
    """Single-use staged readback (compute.d.ts:39-45)."""

    def __init__(self, ctx: "CudaContext", h: int, rows: int, cols: int):
        self._ctx, self._h, self._shape = ctx, h, (rows, cols)

    def read(self, out: Optional[np.ndarray] = None) -> np.ndarray:
        """The snapshot, into `out` (a contiguous f32 array of the right size, e.g. one the caller reuses every
        step) or a new array."""
        if out is None:
            out = np.empty(self._shape[0] * self._shape[1], np.float32)
        assert out.dtype == np.float32 and out.flags["C_CONTIGUOUS"] and out.size >= self._shape[0] * self._shape[1]
        self._ctx._check(self._ctx._lib.fa_staged_read(self._ctx._h, self._h, out.ctypes.data))
        return out


class RecordedBatch:
    """A recorded batch; launch() submits all of its ops with one call."""

    def __init__(self, ctx: "CudaContext", h: int):
        self._ctx, self._h = ctx, h

    def launch(self) -> None:
        self._ctx._check(self._ctx._lib.fa_graph_launch(self._ctx._h, self._h))

    def free(self) -> None:
        if self._h:
            self._ctx._check(self._ctx._lib.fa_graph_free(self._ctx._h, self._h))
            self._h = None


def _np_f32(data) -> np.ndarray:
    return np.ascontiguousarray(data, dtype=np.float32).reshape(-1)


class CudaContext:
    """One compute context = one CUDA stream on one B200 (compute.d.ts:106)."""

    backend = "cuda"
    hasF16 = True

    def __init__(self, device: int = 0):
        self._lib = _lib.load_library()
        h = C.c_void_p()
        rc = self._lib.fa_ctx_create(device, C.byref(h))
        if rc != 0:
            raise CudaError(rc, (self._lib.fa_last_error(None) or b"").decode())
        self._h = h
        self.device = device

    # -- plumbing -------------------------------------------------------------------------
    def _check(self, rc: int):
        if rc != 0:
            raise CudaError(rc, (self._lib.fa_last_error(self._h) or b"").decode())

    def _wrap(self, h: C.c_void_p, view: bool = False) -> Tensor:
        r, c, s = C.c_int(), C.c_int(), C.c_int()
        self._lib.fa_tensor_info(h, C.byref(r), C.byref(c), C.byref(s), None)
        return Tensor(h.value, r.value, c.value, f16=bool(s.value), view=view)

    @staticmethod
    def _h_of(t) -> Optional[int]:
        return None if t is None else t.h

    def _op(self, fn, *args) -> Tensor:
        out = C.c_void_p()
        self._check(fn(self._h, *args, C.byref(out)))
        return self._wrap(out)

    # -- tensors & memory (compute.d.ts:109-133) ------------------------------------------------
    def upload(self, data, rows: int, cols: int) -> Tensor:
        a = _np_f32(data)
        assert a.size >= rows * cols, "upload: data shorter than rows*cols"
        return self._op(self._lib.fa_upload_f32, a.ctypes.data, rows, cols)

    def uploadF16(self, data, rows: int, cols: int) -> Tensor:
        a = _np_f32(data)
        assert a.size >= rows * cols, "uploadF16: data shorter than rows*cols"
        return self._op(self._lib.fa_upload_f16, a.ctypes.data, rows, cols)

    def alloc(self, rows: int, cols: int) -> Tensor:
        return self._op(self._lib.fa_alloc, rows, cols)

    def allocF16(self, rows: int, cols: int) -> Tensor:
        return self._op(self._lib.fa_alloc_f16, rows, cols)

    def ensureTensor(self, t) -> Tensor:
        """Host {data, rows, cols} literal -> tensor; tensors pass through (compute.d.ts:115-117)."""
        if isinstance(t, Tensor):
            return t
        return self.upload(t["data"], t["rows"], t["cols"])

    def uploadBytes(self, typed) -> PackedBytes:
        a = np.ascontiguousarray(typed)
        raw = a.view(np.uint8).reshape(-1)
        out = C.c_void_p()
        self._check(self._lib.fa_upload_bytes(self._h, raw.ctypes.data, raw.size, C.byref(out)))
        return PackedBytes(out.value, raw.size)

    def freeTensor(self, t: Tensor) -> None:
        if t is not None and t.h:
            self._check(self._lib.fa_free_tensor(self._h, t.h))
            t.h = None

    def freeBytes(self, b: PackedBytes) -> None:
        if b is not None and b.h:
            self._check(self._lib.fa_free_bytes(self._h, b.h))
            b.h = None

    def pin(self, t: Tensor, toParent: bool = False) -> Tensor:
        self._check(self._lib.fa_pin(self._h, t.h, 1 if toParent else 0))
        return t

    def pushArena(self) -> int:
        h = C.c_int()
        self._check(self._lib.fa_push_arena(self._h, C.byref(h)))
        return h.value

    def popArena(self, handle: Optional[int] = None) -> None:
        self._check(self._lib.fa_pop_arena(self._h, -1 if handle is None else handle))

    def trimPool(self, budgetBytes: int = 0) -> None:
        self._check(self._lib.fa_trim_pool(self._h, budgetBytes))

    def destroy(self) -> None:
        if self._h:
            self._lib.fa_ctx_destroy(self._h)
            self._h = None
            for p in getattr(self, "_pinned", []):
                self._lib.fa_host_free(p)
            self._pinned = []

    # -- readback (compute.d.ts:135-145) ---------------------------------------------------------
    def download(self, t: Tensor) -> np.ndarray:
        out = np.empty(t.rows * t.cols, np.float32)
        self._check(self._lib.fa_download(self._h, t.h, out.ctypes.data))
        return out

    downloadF16 = download

    def downloadAsync(self, t: Tensor, pinned: np.ndarray) -> None:
        """Enqueue (or record) the device-to-host copy of t into a page-locked array from pinnedArray(); the
        contents are valid after the next sync()."""
        assert pinned.dtype == np.float32 and pinned.flags["C_CONTIGUOUS"] and pinned.size >= t.rows * t.cols
        self._check(self._lib.fa_download_async(self._h, t.h, pinned.ctypes.data))

    def stageDownload(self, t: Tensor) -> StagedRead:
        out = C.c_void_p()
        self._check(self._lib.fa_stage_download(self._h, t.h, C.byref(out)))
        return StagedRead(self, out.value, t.rows, t.cols)

    def rowsView(self, t: Tensor, rows: int) -> Tensor:
        out = C.c_void_p()
        self._check(self._lib.fa_rows_view(self._h, t.h, rows, C.byref(out)))
        return self._wrap(out, view=True)

    def reshapeView(self, t: Tensor, rows: int, cols: int) -> Tensor:
        """Same storage, other [rows, cols] (a JS engine re-labels the tensor object for this)."""
        out = C.c_void_p()
        self._check(self._lib.fa_reshape_view(self._h, t.h, rows, cols, C.byref(out)))
        return self._wrap(out, view=True)

    # -- batching (compute.d.ts:147-151) ----------------------------------------------------------
    def beginBatch(self) -> None:
        self._check(self._lib.fa_begin_batch(self._h))

    def endBatch(self) -> None:
        self._check(self._lib.fa_end_batch(self._h))

    def withBatchSync(self, fn):
        self.beginBatch()
        try:
            return fn()
        finally:
            self.endBatch()

    withBatch = withBatchSync

    def recordBatch(self, fn) -> "RecordedBatch":
        """Record the ops `fn` enqueues into one replayable submission (a CUDA graph) instead of running
        them: the repeatable form of the reference's one-submit batch (src/gpu/scheduler.js:17-60).  Run
        the same sequence once eagerly first so weight repacks and pool growth stay out of the recording.
        Returns (RecordedBatch, whatever fn returned); tensors fn created stay valid across replays."""
        self._check(self._lib.fa_graph_begin(self._h))
        try:
            result = fn()
        except Exception:
            g = C.c_void_p()
            self._lib.fa_graph_end(self._h, C.byref(g))
            if g.value:
                self._lib.fa_graph_free(self._h, g)
            raise
        g = C.c_void_p()
        self._check(self._lib.fa_graph_end(self._h, C.byref(g)))
        return RecordedBatch(self, g.value), result

    # -- linear algebra (compute.d.ts:153-168) -----------------------------------------------------
    def matmul(self, a: Tensor, b: Tensor, opts: Optional[dict] = None, *, bias=None, act="none", add=None) -> Tensor:
        if opts:
            bias, act, add = opts.get("bias", bias), opts.get("act", act), opts.get("add", add)
            if opts.get("operandOnly") and add is None:
                # optional hint: the result is only read as a packed f16 operand (another matmul, attnFusedQKV)
                return self._op(self._lib.fa_matmul_operand, a.h, b.h, self._h_of(bias), ACT[act])
        return self._op(self._lib.fa_matmul, a.h, b.h, self._h_of(bias), ACT[act], self._h_of(add))

    def matmulV2(self, a, b, opts: Optional[dict] = None, *, bias=None, act="none") -> Tensor:
        return self.matmul(a, b, opts, bias=bias, act=act)

    matmulV3 = matmulV4 = matmulF16 = matmulF16C = matmulV2

    def matmulInt8(self, a: Tensor, wq: PackedBytes, scale: Tensor, N: int, K: int, opts: Optional[dict] = None, *,
                   bias=None, act="none") -> Tensor:
        if opts:
            bias, act = opts.get("bias", bias), opts.get("act", act)
        return self._op(self._lib.fa_matmul_int8, a.h, wq.h, scale.h, N, K, self._h_of(bias), ACT[act])

    def matmulInt8Operand(self, a: Tensor, wq: PackedBytes, scale: Tensor, N: int, K: int, opts: Optional[dict] = None, *,
                          bias=None, act="none", add=None, operandOnly=False) -> Tensor:
        """Optional member: matmulInt8 with the weights kept int8 on the device and widened to f16 inside the
        tensor-core kernel; activations rounded to f16 as on matmul's f16-B route; takes a residual `add` and the
        operandOnly hint like matmul."""
        if opts:
            bias, act, add = opts.get("bias", bias), opts.get("act", act), opts.get("add", add)
            operandOnly = opts.get("operandOnly", operandOnly)
        return self._op(self._lib.fa_matmul_int8_operand, a.h, wq.h, scale.h, N, K, self._h_of(bias), ACT[act],
                        self._h_of(add), 1 if operandOnly else 0)

    def matmulNBits(self, a: Tensor, bq: PackedBytes, scales: Tensor, zp: PackedBytes, N: int, blockSize: int = 32) -> Tensor:
        return self._op(self._lib.fa_matmul_nbits, a.h, bq.h, scales.h, zp.h, N, blockSize)

    def int8GemmI32(self, aq: np.ndarray, wq: PackedBytes, N: int, K: int) -> np.ndarray:
        """Integer mode of the int8 tensor-core kernel: exact int32 accumulators [M,N]."""
        aq = np.ascontiguousarray(aq, dtype=np.int8)
        M = aq.shape[0]
        out = np.empty((M, N), np.int32)
        self._check(self._lib.fa_int8_gemm_i32(self._h, aq.ctypes.data, M, wq.h, N, K, out.ctypes.data))
        return out

    def matmulInt8Static(self, a_ptr: int, wq_ptr: int, scale_ptr: int, bias_ptr: Optional[int], act: str, y_ptr: int,
                         M: int, N: int, K: int) -> None:
        """Allocation-free int8 product on raw device pointers (see fa_matmul_int8_static in the header):
        for hosts that cannot allocate device memory when they call.  Scratch is a fixed array inside the
        library; limits M <= 512, K <= 2048, packed weights <= 8 MiB.  Calls must not overlap on the GPU."""
        self._check(self._lib.fa_matmul_int8_static(self._h, a_ptr, wq_ptr, scale_ptr, bias_ptr, ACT[act], y_ptr, M, N, K))

    def layernorm(self, x, gamma, beta, eps: float = 1e-5) -> Tensor:
        return self._op(self._lib.fa_layernorm, x.h, gamma.h, beta.h, eps)

    def layernormOperand(self, x, gamma, beta, eps: float = 1e-5) -> Tensor:
        """Optional member: layernorm whose result the caller only feeds to matmul as the row operand.  For
        many-row inputs it is kept as the packed f16 operand alone; reading it any other way first fills its
        f32 storage from that operand (values rounded to f16)."""
        return self._op(self._lib.fa_layernorm_operand, x.h, gamma.h, beta.h, eps)

    def layernormChain(self, x, g1, b1, g2, b2, eps: float = 1e-5):
        """Optional member: (layernorm(x, g1, b1), layernormOperand(of that, g2, b2)) in one pass over the rows."""
        y, z = C.c_void_p(), C.c_void_p()
        self._check(self._lib.fa_layernorm_chain(self._h, x.h, g1.h, b1.h, g2.h, b2.h, eps, C.byref(y), C.byref(z)))
        return self._wrap(y), self._wrap(z)

    def softmax(self, x) -> Tensor:
        return self._op(self._lib.fa_softmax, x.h)

    # -- convolution (compute.d.ts:170-183) --------------------------------------------------------
    def conv1d(self, x, w, opts: Optional[dict] = None, *, cout=None, k=None, bias=None, stride=1, pad=0, padLeft=None,
               padRight=None, dilation=1, groups=1, act="none") -> Tensor:
        if opts:
            cout, k = opts.get("cout", cout), opts.get("k", k)
            bias, stride, pad = opts.get("bias", bias), opts.get("stride", stride), opts.get("pad", pad)
            padLeft, padRight = opts.get("padLeft", padLeft), opts.get("padRight", padRight)
            dilation, groups, act = opts.get("dilation", dilation), opts.get("groups", groups), opts.get("act", act)
        padLeft = pad if padLeft is None else padLeft
        padRight = pad if padRight is None else padRight
        return self._op(self._lib.fa_conv1d, x.h, w.h, self._h_of(bias), cout, k, stride, padLeft, padRight, dilation,
                        groups, ACT[act])

    def conv1dWindows(self, x, w, opts: dict, windows: int) -> Tensor:
        """conv1d over `windows` independent equal-length column blocks of x in one launch (optional fast
        path for the per-window sliceCols/conv1d/setCols loop of raw-encoder.js:343-351)."""
        pl = opts.get("padLeft", opts.get("pad", 0))
        pr = opts.get("padRight", opts.get("pad", 0))
        assert opts.get("stride", 1) == 1
        return self._op(self._lib.fa_conv1d_windows, x.h, w.h, self._h_of(opts.get("bias")), opts["cout"], opts["k"], pl, pr,
                        opts.get("dilation", 1), opts.get("groups", 1), ACT[opts.get("act", "none")], windows)

    def gluDwConvTimeMajor(self, x, w, opts: dict, windows: int) -> Tensor:
        """transpose -> glu -> per-window depthwise conv1d(+act) -> transpose of the conformer conv module
        (raw-encoder.js:340-362) in one launch, time-major in and out: x [W*T, 2D] -> [W*T, D]."""
        pl = opts.get("padLeft", opts.get("pad", 0))
        pr = opts.get("padRight", opts.get("pad", 0))
        return self._op(self._lib.fa_glu_dwconv_tm, x.h, w.h, self._h_of(opts.get("bias")), opts["k"], pl, pr,
                        ACT[opts.get("act", "none")], windows)

    def conv2d(self, x, weight, opts: Optional[dict] = None, **kw) -> Tensor:
        o = dict(opts or {})
        o.update(kw)
        padH, padW = o.get("padH", 0), o.get("padW", 0)
        pt = o.get("padTop", padH) if o.get("padTop") is not None else padH
        pb = o.get("padBottom", padH) if o.get("padBottom") is not None else padH
        pl = o.get("padLeft", padW) if o.get("padLeft") is not None else padW
        pr = o.get("padRight", padW) if o.get("padRight") is not None else padW
        return self._op(self._lib.fa_conv2d, x.h, weight.h, self._h_of(o.get("bias")), o["cout"], o["cin"], o["h"], o["w"],
                        o["kh"], o["kw"], o.get("strideH", 1), o.get("strideW", 1), pt, pb, pl, pr, o.get("groups", 1),
                        ACT[o.get("act", "none")])

    def conv2dWindows(self, x, weight, opts: dict, W: int) -> Tensor:
        """conv2d over W images at once: x [W, cin*h*w] -> [W, cout*Ho*Wo] (optional member)."""
        o = dict(opts)
        padH, padW = o.get("padH", 0), o.get("padW", 0)
        pt = o.get("padTop", padH) if o.get("padTop") is not None else padH
        pb = o.get("padBottom", padH) if o.get("padBottom") is not None else padH
        pl = o.get("padLeft", padW) if o.get("padLeft") is not None else padW
        pr = o.get("padRight", padW) if o.get("padRight") is not None else padW
        return self._op(self._lib.fa_conv2d_windows, x.h, weight.h, self._h_of(o.get("bias")), o["cout"], o["cin"], o["h"],
                        o["w"], o["kh"], o["kw"], o.get("strideH", 1), o.get("strideW", 1), pt, pb, pl, pr, o.get("groups", 1),
                        ACT[o.get("act", "none")], W)

    def subReshapeWindows(self, x, Cc: int, Tsub: int, F: int, W: int) -> Tensor:
        """subReshape over W windows at once: x [W, C*Tsub*F] -> [W*Tsub, C*F] (optional member)."""
        return self._op(self._lib.fa_sub_reshape_windows, x.h, Cc, Tsub, F, W)

    def convStemWindows(self, x, layers, Cc: int, h: int, w: int, W: int) -> Optional[Tensor]:
        """Optional member: the stem's first three layers (3x3 stride-2 conv from one channel + relu, 3x3 stride-2
        depthwise, pointwise + relu) over W images x [W, h*w] in one call; `layers` = three dicts {"w", "b"}.
        Returns [W, C*H2*W2], bit-identical to the three conv2dWindows calls, or None when the geometry is
        outside the fused kernel's range (the caller then makes those calls)."""
        out = C.c_void_p()
        hs = []
        for l in layers:
            hs += [l["w"].h, self._h_of(l.get("b"))]
        self._check(self._lib.fa_conv_stem_windows(self._h, x.h, *hs, Cc, h, w, W, C.byref(out)))
        return self._wrap(out) if out.value else None

    def convDwPwWindows(self, x, layers, Cc: int, h: int, w: int, W: int) -> Optional[Tensor]:
        """Optional member: 3x3 stride-2 depthwise conv then pointwise conv + relu over W feature maps
        x [W, C*h*w] in one call; `layers` = two dicts {"w", "b"}.  Bit-identical to the two conv2dWindows calls;
        None outside the fused kernel's range (w == 32, C a multiple of 64)."""
        out = C.c_void_p()
        hs = []
        for l in layers:
            hs += [l["w"].h, self._h_of(l.get("b"))]
        self._check(self._lib.fa_conv_dw_pw_windows(self._h, x.h, *hs, Cc, h, w, W, C.byref(out)))
        return self._wrap(out) if out.value else None

    # -- attention (compute.d.ts:189-199) ----------------------------------------------------------
    def bmmQK(self, q, b, qb, H: int, HD: int, W: int = 1, bShared: bool = False) -> Tensor:
        return self._op(self._lib.fa_bmm_qk, q.h, b.h, self._h_of(qb), H, HD, W, 1 if bShared else 0)

    def bmmPV(self, p, v, H: int, HD: int, W: int = 1) -> Tensor:
        return self._op(self._lib.fa_bmm_pv, p.h, v.h, H, HD, W)

    def attnFused(self, q, k, v, pos, pbu, pbv, H: int, HD: int, W: int) -> Optional[Tensor]:
        """Fused rel-pos self-attention (optional member, compute.d.ts:247-248).  Returns None when the
        shape is outside the fused kernel's range - the caller then runs the separate ops."""
        out = C.c_void_p()
        self._check(self._lib.fa_attn_fused(self._h, q.h, k.h, v.h, pos.h, pbu.h, pbv.h, H, HD, W, C.byref(out)))
        return self._wrap(out) if out.value else None

    def attnFusedQKV(self, qkv, pos, pbu, pbv, H: int, HD: int, W: int) -> Optional[Tensor]:
        """Optional member: attnFused over one fused projection qkv [W*T, 3*H*HD] (q | k | v columns).  Returns
        None outside the one-kernel form's range (HD == 128, 16 <= T <= 192)."""
        out = C.c_void_p()
        self._check(self._lib.fa_attn_fused_qkv(self._h, qkv.h, pos.h, pbu.h, pbv.h, H, HD, W, C.byref(out)))
        return self._wrap(out) if out.value else None

    def relShift(self, x) -> Tensor:
        return self._op(self._lib.fa_rel_shift_b, x.h, 1)

    def relShiftB(self, x, H: int) -> Tensor:
        return self._op(self._lib.fa_rel_shift_b, x.h, H)

    # -- elementwise & data movement (compute.d.ts:201-224) -----------------------------------------
    def ewise(self, a, b, op: str) -> Tensor:
        return self._op(self._lib.fa_ewise, a.h, b.h, 1 if op == "mul" else 0)

    def add(self, a, b) -> Tensor:
        return self.ewise(a, b, "add")

    def mul(self, a, b) -> Tensor:
        return self.ewise(a, b, "mul")

    def scale(self, x, s: float) -> Tensor:
        return self._op(self._lib.fa_scale, x.h, float(s))

    def silu(self, x) -> Tensor:
        return self._op(self._lib.fa_unary, x.h, ACT["silu"])

    def relu(self, x) -> Tensor:
        return self._op(self._lib.fa_unary, x.h, ACT["relu"])

    def glu(self, x) -> Tensor:
        return self._op(self._lib.fa_glu, x.h)

    def transpose(self, x) -> Tensor:
        return self._op(self._lib.fa_transpose, x.h)

    def sliceCols(self, x, col0: int, width: int) -> Tensor:
        return self._op(self._lib.fa_slice_cols, x.h, col0, width)

    def setCols(self, dst, src, col0: int) -> Tensor:
        self._check(self._lib.fa_set_cols(self._h, dst.h, src.h, col0))
        return dst

    def sliceRows(self, x, row0: int, count: int) -> Tensor:
        return self._op(self._lib.fa_slice_rows, x.h, row0, count)

    def copyRows(self, dst, src, rowOffset: int) -> Tensor:
        self._check(self._lib.fa_copy_rows(self._h, dst.h, src.h, rowOffset))
        return dst

    def concatRows(self, tensors: Sequence[Tensor]) -> Tensor:
        arr = (C.c_void_p * len(tensors))(*[t.h for t in tensors])
        return self._op(self._lib.fa_concat_rows, arr, len(tensors))

    def subReshape(self, x, Cc: int, Tsub: int, F: int) -> Tensor:
        return self._op(self._lib.fa_sub_reshape, x.h, Cc, Tsub, F)

    def argmaxRowsIndex(self, x, ncols: int = 0) -> Tensor:
        """[rows, 2] = {argmax index, max value} per row over the first `ncols` columns (0 = all); the
        host token pick moved to the device."""
        return self._op(self._lib.fa_argmax_rows, x.h, ncols)

    def unshardCols(self, gathered: Tensor, world: int) -> Tensor:
        """[world*M, Ns] column shards stacked along rows -> the row-major [M, world*Ns] product."""
        return self._op(self._lib.fa_unshard_cols, gathered.h, world)

    # -- peer mappings and the product with a fused all-gather (one process per GPU) ----------------------
    def ipcExport(self, t: Tensor) -> bytes:
        buf = (C.c_ubyte * 64)()
        self._check(self._lib.fa_ipc_export(self._h, t.h, buf))
        return bytes(buf)

    def ipcOpen(self, handle: bytes) -> int:
        buf = (C.c_ubyte * 64).from_buffer_copy(handle)
        out = C.c_void_p()
        self._check(self._lib.fa_ipc_open(self._h, buf, C.byref(out)))
        return out.value

    def ipcClose(self, ptr: int) -> None:
        self._check(self._lib.fa_ipc_close(self._h, C.c_void_p(ptr)))

    def matmulScatter(self, a: Tensor, b_shard: Tensor, out_ptrs, ldc: int, col0: int, *, bias=None, act="none") -> None:
        """This rank's block of output columns written into every buffer of `out_ptrs` (own first, then the
        peers' IPC mappings) by the product's own epilogue."""
        arr = (C.c_void_p * len(out_ptrs))(*[C.c_void_p(int(p)) for p in out_ptrs])
        self._check(self._lib.fa_matmul_scatter(self._h, a.h, b_shard.h, self._h_of(bias), ACT[act], arr, len(out_ptrs), ldc, col0))

    def logMelWindows(self, audio: Tensor, nMels: int = 128, logGuard: float = 2.0 ** -24, normalize: bool = True) -> Tensor:
        """Optional member: the reference's host-side log-mel front end (ParakeetMel / JsPreprocessor,
        src/engines/asr-parakeet/parakeet-mel.js, src/engines/asr-nemotron/nemotron-mel.js) for a batch of windows
        on the device.  audio [W, N] f32 at 16 kHz -> [W, T*nMels], time-major per window, T = floor(N/160)
        (normalize=True, Parakeet) or N/160 + 1 (normalize=False with logGuard=1e-10, Nemotron)."""
        return self._op(self._lib.fa_log_mel_windows, audio.h, int(nMels), float(logGuard), 1 if normalize else 0)

    def embedRows(self, table: Tensor, pos: Tensor, idx: Tensor, n: int) -> Tensor:
        """[S, D] = table[id_s] + pos[n], ids read from column 0 of `idx` on the device (so a greedy
        decode needs no host round trip between tokens)."""
        return self._op(self._lib.fa_embed_rows, table.h, pos.h, idx.h, n)

    # -- profiling / stats (compute.d.ts:250-254) --------------------------------------------------
    def startProfile(self, maxOps: int = 4096) -> None:
        self._check(self._lib.fa_profile_start(self._h, maxOps))

    def endProfile(self):
        cap = 256
        buf = (_lib.ProfileEntry * cap)()
        n = C.c_int()
        self._check(self._lib.fa_profile_end(self._h, buf, cap, C.byref(n)))
        return [{"label": buf[i].label.decode(), "ms": buf[i].ms, "count": buf[i].count} for i in range(min(n.value, cap))]

    def memStats(self):
        a, b, c, d = (C.c_ulonglong() for _ in range(4))
        self._check(self._lib.fa_mem_stats(self._h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
        return {"created": a.value, "createdBytes": b.value, "reused": c.value, "poolBytes": d.value}

    def poolInfo(self):
        return {"bytes": self.memStats()["poolBytes"]}

    # -- extras for harnesses ------------------------------------------------------------------
    def mark(self) -> None:
        """Record a point in this context's stream (all that was enqueued so far) that other contexts can wait for."""
        self._check(self._lib.fa_ctx_mark(self._h))

    def waitMark(self, other: "CudaContext") -> None:
        """What this context enqueues from now on waits, on the device, for the point `other` marked last."""
        self._check(self._lib.fa_ctx_wait_mark(self._h, other._h))

    def sync(self) -> None:
        self._check(self._lib.fa_sync(self._h))

    def launchCount(self) -> int:
        n = C.c_ulonglong()
        self._check(self._lib.fa_launch_count(self._h, C.byref(n)))
        return n.value

    def setOption(self, key: str, value: int) -> None:
        self._check(self._lib.fa_ctx_set_option(self._h, key.encode(), int(value)))

    def pinnedArray(self, n_floats: int) -> np.ndarray:
        """Page-locked host f32 buffer (uploads from it and downloads into it are asynchronous copies)."""
        p = C.c_void_p()
        self._check(self._lib.fa_host_alloc(max(1, n_floats) * 4, C.byref(p)))
        arr = np.ctypeslib.as_array((C.c_float * max(1, n_floats)).from_address(p.value))
        self._pinned = getattr(self, "_pinned", [])
        self._pinned.append(p)
        return arr[:n_floats]

    def stream(self) -> int:
        s = C.c_void_p()
        self._check(self._lib.fa_ctx_stream(self._h, C.byref(s)))
        return s.value or 0

    def devicePtr(self, t: Tensor) -> int:
        p = C.c_void_p()
        self._check(self._lib.fa_tensor_ptr(self._h, t.h, C.byref(p)))
        return p.value or 0


def create_context(backend: str = "cuda", device: int = 0) -> CudaContext:
    """The "cuda" branch a maintainer adds to createContext() (src/gpu/context.js:23-37)."""
    if backend != "cuda":
        raise ValueError(f"this package only provides the 'cuda' backend (asked for {backend!r})")
    return CudaContext(device)
