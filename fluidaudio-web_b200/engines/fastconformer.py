"""FastConformer (Parakeet-TDT-0.6B-shaped) encoder forward, op for op the sequence of
src/engines/asr-parakeet/raw-encoder.js (loadParakeetEncoder :39-161, posEncoding :163-175,
preEncode :177-222, parakeetEncodeBatch :235-386), written only against ComputeContext members.

Arch: mel[melBins, T] -> dw-striding 8x subsampling (conv2d x5) -> linear -> N x conformer block
(macaron FF half, rel-pos MHSA, conv module, FF half, LayerNorm).  Folded into weights at load:
q * 1/sqrt(HD), pos_bias_u/v * 1/sqrt(HD), FF output projections * 0.5.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np


def infer_config(man: Dict[str, np.ndarray]) -> dict:
    """raw-encoder.js:28-35: every size is read off the weight shapes."""
    layers = sum(1 for k in man if k.endswith("_lnff1_w"))
    D, DFF = man["L0_ff1w1"].shape
    H, HD = man["L0_pbu"].shape
    Csub = man["c0w"].shape[0]
    Fsub = man["linw"].shape[0] // Csub
    return dict(D=D, DFF=DFF, H=H, HD=HD, layers=layers, dwK=man["L0_dw"].shape[2], Csub=Csub, Fsub=Fsub,
                melBins=Fsub * 8)


class Int8Weight:
    """A weight matrix [K, N] kept int8 on the device with its per-output-column f32 scales (optional backend member
    matmulInt8Operand); `rows` / `cols` mirror a tensor's so that shape inference keeps working."""

    __slots__ = ("q", "scale", "rows", "cols")

    def __init__(self, ctx, q_kn: np.ndarray, scale: np.ndarray):
        self.rows, self.cols = q_kn.shape
        self.q = ctx.uploadBytes(np.ascontiguousarray(q_kn, np.int8))
        self.scale = ctx.upload(np.ascontiguousarray(scale, np.float32), 1, scale.size)


def mm(ctx, x, w, opts: Optional[dict] = None):
    """matmul against a weight that is either a backend tensor (f16 storage) or an Int8Weight."""
    if isinstance(w, Int8Weight):
        return ctx.matmulInt8Operand(x, w.q, w.scale, w.cols, w.rows, opts)
    return ctx.matmul(x, w, opts)


def load_encoder_blob(ctx, blob: bytes, man: dict, int8_resident: bool = True, cfg_override: Optional[dict] = None) -> dict:
    """loadParakeetEncoder for the int8 artifact (raw-encoder.js:39-161; format: engines/blob.py).  With
    int8_resident the matrices the artifact stores int8 per output column (and the two pointwise convolutions, stored
    per output channel = per column of their transposed form) stay int8 on the device - half the bytes of the f16
    storage the reference uploads - and run through the backend's optional member matmulInt8Operand; the folds of the
    loader (q * 1/sqrt(HD), FF output projections * 0.5) go into the column scales, exactly.  Without it (or on a
    backend without that member) every tensor is dequantised on the host as the reference does."""
    from . import blob as blobfmt

    b = blobfmt.Blob(blob, man)
    weights = b.as_f32_dict()
    if not (int8_resident and hasattr(ctx, "matmulInt8Operand")):
        return load_encoder(ctx, weights, cfg_override)
    return load_encoder(ctx, weights, cfg_override, _i8=b)


def load_encoder(ctx, weights: Dict[str, np.ndarray], cfg_override: Optional[dict] = None, _i8=None) -> dict:
    """Upload all encoder weights once (raw-encoder.js:39-161).  `weights` holds f32 arrays (already
    dequantised when the artifact stores int8, :55-76).  Matrices go up as f16 storage (:92-95)."""
    cfg = {**infer_config(weights), **(cfg_override or {})}
    HD, D = cfg["HD"], cfg["D"]
    INV = 1.0 / math.sqrt(HD)
    f32 = np.float32

    def mat(k, s=None):
        if _i8 is not None and _i8.is_i8(k) and _i8.man[k]["quant"] == "col":
            q, sc, _ = _i8.tensor_i8(k)  # stays int8; a fold multiplies the column scales
            return Int8Weight(ctx, q, sc if s is None else (sc * f32(s)).astype(f32))
        a = weights[k].astype(f32)
        if s is not None:
            a = (a * f32(s)).astype(f32)
        return ctx.uploadF16(a, a.shape[0], a.shape[1])

    def vec(k, s=None):
        a = weights[k].astype(f32).reshape(-1)
        if s is not None:
            a = (a * f32(s)).astype(f32)
        return ctx.upload(a, 1, a.size)

    def vec_opt(k, s=None):
        return vec(k, s) if k in weights else None

    def pwT(k, cout, cin):
        # pointwise conv weight [cout, cin, 1] as a transposed matrix [cin, cout] (:112-118)
        if _i8 is not None and _i8.is_i8(k):
            q, sc, _ = _i8.tensor_i8(k)  # per-output-channel scales = per column of the transposed matrix
            return Int8Weight(ctx, np.ascontiguousarray(q.reshape(cout, cin).T), sc)
        w = weights[k].astype(f32).reshape(cout, cin)
        return ctx.uploadF16(np.ascontiguousarray(w.T), cin, cout)

    sub = dict(conv=[dict(w=vec(f"c{i}w"), b=vec(f"c{i}b")) for i in range(5)], linw=mat("linw"), linb=vec("linb"))
    layers = []
    for L in range(cfg["layers"]):
        g = lambda s: f"L{L}_{s}"
        layers.append(dict(
            lnff1=(vec(g("lnff1_w")), vec(g("lnff1_b"))), ff1w1=mat(g("ff1w1")), ff1w2=mat(g("ff1w2"), 0.5),
            ff1b1=vec_opt(g("ff1b1")), ff1b2=vec_opt(g("ff1b2"), 0.5),
            lnatt=(vec(g("lnatt_w")), vec(g("lnatt_b"))), q=mat(g("q"), INV), k=mat(g("k")), v=mat(g("v")),
            pos=mat(g("pos")), out=mat(g("out")), qb=vec_opt(g("qb"), INV), kb=vec_opt(g("kb")), vb=vec_opt(g("vb")),
            outb=vec_opt(g("outb")), pbuAll=vec(g("pbu"), INV), pbvAll=vec(g("pbv"), INV),
            lnconv=(vec(g("lnconv_w")), vec(g("lnconv_b"))), pw1T=pwT(g("pw1"), 2 * D, D), dw=vec(g("dw")),
            dwb=vec(g("dwb")), pw2T=pwT(g("pw2"), D, D), pw1b=vec_opt(g("pw1b")), pw2b=vec_opt(g("pw2b")),
            lnff2=(vec(g("lnff2_w")), vec(g("lnff2_b"))), ff2w1=mat(g("ff2w1")), ff2w2=mat(g("ff2w2"), 0.5),
            ff2b1=vec_opt(g("ff2b1")), ff2b2=vec_opt(g("ff2b2"), 0.5), lnout=(vec(g("lnout_w")), vec(g("lnout_b")))))
    if hasattr(ctx, "attnFusedQKV") and HD == 128:
        # optional member: q | k | v as ONE projection (weights and biases side by side), consumed column-wise
        for L, lw in enumerate(layers):
            g = lambda s: f"L{L}_{s}"
            if _i8 is not None and all(_i8.is_i8(g(n)) for n in "qkv"):
                qs = [_i8.tensor_i8(g(n)) for n in "qkv"]
                lw["qkv"] = Int8Weight(ctx, np.concatenate([t[0] for t in qs], axis=1),
                                       np.concatenate([(qs[0][1] * f32(INV)).astype(f32), qs[1][1], qs[2][1]]))
                cat = np.zeros((1, 3 * weights[g("q")].shape[1]), f32)
            else:
                cat = np.concatenate([weights[g("q")].astype(f32) * f32(INV), weights[g("k")].astype(f32),
                                      weights[g("v")].astype(f32)], axis=1).astype(f32)
                lw["qkv"] = ctx.uploadF16(np.ascontiguousarray(cat), cat.shape[0], cat.shape[1])
            n = cat.shape[1] // 3
            parts = [(g("qb"), INV), (g("kb"), None), (g("vb"), None)]
            if any(k in weights for k, _ in parts):
                b = np.zeros(3 * n, f32)
                for i, (k, sc) in enumerate(parts):
                    if k in weights:
                        v = weights[k].astype(f32).reshape(-1)
                        b[i * n:(i + 1) * n] = (v * f32(sc)).astype(f32) if sc is not None else v
                lw["qkvb"] = ctx.upload(b, 1, b.size)
            else:
                lw["qkvb"] = None
    return dict(sub=sub, layers=layers, cfg=cfg, _pe={}, _posProj={})


def pos_encoding(Tsub: int, D: int) -> np.ndarray:
    """raw-encoder.js:163-175 (computed in doubles, stored f32)."""
    pos = (Tsub - 1 - np.arange(2 * Tsub - 1, dtype=np.float64))[:, None]
    i = np.arange(0, D, 2, dtype=np.float64)
    dv = np.exp(i * -(math.log(10000.0) / D))[None, :]
    pe = np.empty((2 * Tsub - 1, D), np.float32)
    pe[:, 0::2] = np.sin(pos * dv)
    pe[:, 1::2] = np.cos(pos * dv)
    return pe


def mel_time_major(mel: np.ndarray, melBins: int) -> np.ndarray:
    """The host-side transpose of preEncode (:181-183): mel [melBins*T] channel-major -> [T*melBins]."""
    Tfull = mel.size // melBins
    return np.ascontiguousarray(mel.reshape(melBins, Tfull).T, dtype=np.float32).reshape(-1)


def pre_encode(ctx, enc, mel):
    """Subsampling + linear for ONE window -> x [Tsub, D] (:177-222).  `mel` is the reference's
    channel-major array [melBins*T], or a backend tensor [1, T*melBins] that already holds the
    time-major image (so a caller can keep windows resident on the device)."""
    cfg = enc["cfg"]
    Csub, melBins = cfg["Csub"], cfg["melBins"]
    if isinstance(mel, np.ndarray):
        s = ctx.upload(mel_time_major(mel, melBins), 1, mel.size)
    else:
        s = mel
    Tfull = (s.rows * s.cols) // melBins
    Hh, Wd = Tfull, melBins
    conv = [(Csub, 1, 3, 2, 1, "relu", True), (Csub, Csub, 3, 2, Csub, "none", True), (Csub, Csub, 1, 1, 1, "relu", False),
            (Csub, Csub, 3, 2, Csub, "none", True), (Csub, Csub, 1, 1, 1, "relu", False)]
    for i, (cout, cin, k, st, gr, act, s2) in enumerate(conv):
        p = 1 if s2 else 0
        s = ctx.conv2d(s, enc["sub"]["conv"][i]["w"], dict(cout=cout, cin=cin, h=Hh, w=Wd, kh=k, kw=k,
                                                          bias=enc["sub"]["conv"][i]["b"], strideH=st, strideW=st,
                                                          padTop=p, padBottom=p, padLeft=p, padRight=p, groups=gr, act=act))
        Hh = (Hh + 2 * p - k) // st + 1
        Wd = (Wd + 2 * p - k) // st + 1
    flat = ctx.subReshape(s, Csub, Hh, Wd)
    return mm(ctx, flat, enc["sub"]["linw"], dict(bias=enc["sub"]["linb"])), Hh


def pre_encode_windows(ctx, enc, mels):
    """pre_encode for W equal-length windows in one pass of window-batched launches (optional members
    conv2dWindows / subReshapeWindows): same per-window arithmetic, x [W*Tsub, D] directly."""
    cfg = enc["cfg"]
    Csub, melBins = cfg["Csub"], cfg["melBins"]
    if not isinstance(mels, (list, tuple)):  # one backend tensor [W, T*melBins], a time-major window per row
        s, W = mels, mels.rows               # (what the optional member logMelWindows returns)
    elif isinstance(mels[0], np.ndarray):
        W = len(mels)
        stacked = np.stack([mel_time_major(m, melBins) for m in mels])
        s = ctx.upload(stacked, W, stacked.shape[1])
    else:
        W = len(mels)
        s = ctx.concatRows(list(mels))  # [W, T*melBins]
    Hh, Wd = s.cols // melBins, melBins
    conv = [(Csub, 1, 3, 2, 1, "relu", True), (Csub, Csub, 3, 2, Csub, "none", True), (Csub, Csub, 1, 1, 1, "relu", False),
            (Csub, Csub, 3, 2, Csub, "none", True), (Csub, Csub, 1, 1, 1, "relu", False)]
    first = 0
    if hasattr(ctx, "convStemWindows"):  # optional member: layers 0-2 without storing the two largest feature maps
        head = ctx.convStemWindows(s, enc["sub"]["conv"][:3], Csub, Hh, Wd, W)
        if head is not None:
            s, first = head, 3
            Hh, Wd = ((Hh - 1) // 2 + 1 - 1) // 2 + 1, ((Wd - 1) // 2 + 1 - 1) // 2 + 1
    if first == 3 and hasattr(ctx, "convDwPwWindows"):  # optional member: layers 3-4, no f32 depthwise result, no pack pass
        tail = ctx.convDwPwWindows(s, enc["sub"]["conv"][3:5], Csub, Hh, Wd, W)
        if tail is not None:
            s, first = tail, 5
            Hh, Wd = (Hh - 1) // 2 + 1, (Wd - 1) // 2 + 1
    for i, (cout, cin, k, st, gr, act, s2) in enumerate(conv):
        if i < first:
            continue
        p = 1 if s2 else 0
        s = ctx.conv2dWindows(s, enc["sub"]["conv"][i]["w"], dict(cout=cout, cin=cin, h=Hh, w=Wd, kh=k, kw=k,
                                                                 bias=enc["sub"]["conv"][i]["b"], strideH=st, strideW=st,
                                                                 padTop=p, padBottom=p, padLeft=p, padRight=p, groups=gr,
                                                                 act=act), W)
        Hh = (Hh + 2 * p - k) // st + 1
        Wd = (Wd + 2 * p - k) // st + 1
    flat = ctx.subReshapeWindows(s, Csub, Hh, Wd, W)
    return mm(ctx, flat, enc["sub"]["linw"], dict(bias=enc["sub"]["linb"])), Hh


def encode_batch(ctx, enc, mels: List[np.ndarray], layer_hook=None, use_fast: bool = True):
    """W same-length windows concatenated along rows (:235-386): GEMMs see M = W*Tsub, attention and the
    depthwise conv stay per window.  Optional backend members (feature-tested, like the reference tests
    `ctx.attnFused`) replace per-window loops when `use_fast`; use_fast=False is the reference's exact op
    sequence.  Returns (frames [W*Tsub, D], Tsub)."""
    cfg = enc["cfg"]
    D, H, HD, LAYERS, dwK = cfg["D"], cfg["H"], cfg["HD"], cfg["layers"], cfg["dwK"]
    ln = lambda x, lp: ctx.layernorm(x, lp[0], lp[1])
    if not isinstance(mels, (list, tuple)):  # stacked windows on the device (see pre_encode_windows)
        if not (hasattr(ctx, "conv2dWindows") and hasattr(ctx, "subReshapeWindows") and mels.rows > 1):
            mels = [ctx.sliceRows(mels, i, 1) for i in range(mels.rows)]
    W = mels.rows if not isinstance(mels, (list, tuple)) else len(mels)
    sizes = {0} if not isinstance(mels, (list, tuple)) else {(m.size if isinstance(m, np.ndarray) else m.rows * m.cols) for m in mels}
    if use_fast and W > 1 and len(sizes) == 1 and hasattr(ctx, "conv2dWindows") and hasattr(ctx, "subReshapeWindows"):
        x, Tsub = pre_encode_windows(ctx, enc, mels)  # optional members: the whole front end in 7 launches
    else:
        pre = [pre_encode(ctx, enc, m) for m in mels]
        Tsub = pre[0][1]
        if any(p[1] != Tsub for p in pre):
            raise ValueError("encode_batch: windows must have equal Tsub")
        x = pre[0][0] if W == 1 else ctx.concatRows([p[0] for p in pre])
    peT = enc["_pe"].get(Tsub)
    if peT is None:
        peT = ctx.upload(pos_encoding(Tsub, D), 2 * Tsub - 1, D)
        enc["_pe"][Tsub] = peT
    dwPadL = dwPadR = (dwK - 1) >> 1

    # a layernorm that only feeds products: optional member, keeps the result as the product's operand alone
    ln_op = (lambda x, lp: ctx.layernormOperand(x, lp[0], lp[1])) if use_fast and hasattr(ctx, "layernormOperand") else ln

    def ff(x, lp, w1, w2, b1, b2, xn=None):
        xn = ln_op(x, lp) if xn is None else xn
        return mm(ctx, mm(ctx, xn, w1, dict(bias=b1, act="silu")), w2, dict(bias=b2, add=x))

    # optional member: a block's last layernorm and the next block's first one in one pass over the rows
    chain = use_fast and hasattr(ctx, "layernormChain")

    def body():
        nonlocal x
        xff = None  # layernorm(x, lnff1) of the coming block when the previous block already made it
        for L in range(LAYERS):
            layerArena = ctx.pushArena()
            try:
                w = enc["layers"][L]
                x = ff(x, w["lnff1"], w["ff1w1"], w["ff1w2"], w["ff1b1"], w["ff1b2"], xff)
                xff = None
                xln = ln_op(x, w["lnatt"])
                fused_qkv = use_fast and "qkv" in w and W * Tsub >= 256 and 16 <= Tsub <= 192
                if fused_qkv:
                    qkv = mm(ctx, xln, w["qkv"], dict(bias=w["qkvb"], operandOnly=True))  # read by attnFusedQKV only
                else:
                    q = mm(ctx, xln, w["q"], dict(bias=w["qb"]))
                    k = mm(ctx, xln, w["k"], dict(bias=w["kb"]))
                    v = mm(ctx, xln, w["v"], dict(bias=w["vb"]))
                if W > 1:  # pos projection is constant per (layer, Tsub): cached across groups (:307-317)
                    p = enc["_posProj"].get((L, Tsub))
                    if p is None:
                        p = ctx.pin(mm(ctx, peT, w["pos"]))
                        enc["_posProj"][(L, Tsub)] = p
                else:
                    p = mm(ctx, peT, w["pos"])
                outc = None
                if fused_qkv:
                    outc = ctx.attnFusedQKV(qkv, p, w["pbuAll"], w["pbvAll"], H, HD, W)
                    if outc is None:  # declined: cut the columns apart and carry on with the separate members
                        S = H * HD
                        q, k, v = (ctx.sliceCols(qkv, i * S, S) for i in range(3))
                if outc is None and use_fast and getattr(ctx, "attnFused", None):  # optional member, may decline (:333-336)
                    outc = ctx.attnFused(q, k, v, p, w["pbuAll"], w["pbvAll"], H, HD, W)
                if outc is None:
                    ac = ctx.bmmQK(q, k, w["pbuAll"], H, HD, W)
                    bd = ctx.relShiftB(ctx.bmmQK(q, p, w["pbvAll"], H, HD, W, True), W * H)
                    probs = ctx.softmax(ctx.add(ac, bd))
                    outc = ctx.bmmPV(probs, v, H, HD, W)
                x = mm(ctx, outc, w["out"], dict(bias=w["outb"], add=x))
                pre1 = mm(ctx, ln_op(x, w["lnconv"]), w["pw1T"], dict(bias=w["pw1b"]))  # [W*T, 2D]
                opts = dict(cout=D, k=dwK, groups=D, padLeft=dwPadL, padRight=dwPadR, bias=w["dwb"], act="silu")
                if use_fast and hasattr(ctx, "gluDwConvTimeMajor"):  # optional member: the module's middle in one launch
                    dwoT = ctx.gluDwConvTimeMajor(pre1, w["dw"], opts, W)  # [W*T, D]
                else:
                    glu = ctx.glu(ctx.transpose(pre1))  # [D, W*T]
                    if W == 1:
                        dwo = ctx.conv1d(glu, w["dw"], opts)
                    elif use_fast and hasattr(ctx, "conv1dWindows"):  # optional member: all windows in one launch
                        dwo = ctx.conv1dWindows(glu, w["dw"], opts, W)
                    else:  # depthwise conv is over time -> per window (:343-351)
                        dwo = ctx.alloc(D, W * Tsub)
                        for wi in range(W):
                            ctx.setCols(dwo, ctx.conv1d(ctx.sliceCols(glu, wi * Tsub, Tsub), w["dw"], opts), wi * Tsub)
                    dwoT = ctx.transpose(dwo)
                x = mm(ctx, dwoT, w["pw2T"], dict(bias=w["pw2b"], add=x))
                x = ff(x, w["lnff2"], w["ff2w1"], w["ff2w2"], w["ff2b1"], w["ff2b2"])
                if chain and L + 1 < LAYERS:
                    nxt = enc["layers"][L + 1]["lnff1"]
                    x, xff = ctx.layernormChain(x, w["lnout"][0], w["lnout"][1], nxt[0], nxt[1])
                    ctx.pin(xff, True)
                else:
                    x = ln(x, w["lnout"])
                ctx.pin(x, True)  # x feeds the next layer: promote to the enclosing arena
                if layer_hook is not None:
                    layer_hook(L, x)
            finally:
                ctx.popArena(layerArena)
        return x

    return ctx.withBatchSync(body), Tsub


class PipelinedEncoder:
    """encode_batch for a stream of window batches with the host<->device copies hidden: `depth` contexts (one
    CUDA stream each) on one GPU take the batches in turn.  A slot holds two recordings - the upload of the batch's
    windows from page-locked host memory (with the log-mel front end when the windows are PCM), and the forward - and
    reads the frames back into a page-locked result array behind them.  The forwards of different slots are ordered on the device (each waits for the point the slot
    before it marked behind its forward), so that one forward has the whole GPU at a time, while the copies of a
    batch run under the forward of another and the host never copies a frame.  (Two whole forwards left to run side
    by side take each other's SMs kernel by kernel: every persistent product then runs on what the other leaves.)
    submit() launches one batch and hands back the frames of the batch submitted `depth - 1` calls earlier (None
    until the pipeline is full) as a view of that slot's result array: valid until the next submit(), which
    re-launches that slot.  flush() drains the pipeline and returns copies.

    ctxs: the contexts; encs: load_encoder(ctx, weights) for each; host_windows(slot): the list of page-locked
    f32 arrays (time-major windows, see mel_time_major) that slot's recording uploads on every launch - the caller
    fills them before submit()."""

    def __init__(self, ctxs, encs, host_windows, mel_len: int, from_pcm: bool = False, post=None, resident=None, read_back: bool = True):
        """from_pcm: the host windows hold 16 kHz PCM (mel_len = samples per window) and the recording starts with the
        log-mel front end on the device (optional member logMelWindows; the reference runs it in host workers,
        src/engines/asr-parakeet/mel-scheduler.js).  post(slot, frames) -> tensor: an op riding the batch whose result
        is read back instead of the frames (the joint's encoder projection, src/engines/asr-parakeet/pipeline.js:57-61).
        resident: one device tensor of features per slot, in place of host windows (nothing is uploaded).
        read_back=False: the result stays on the device (self.outs[slot]) for a consumer on the slot's stream."""
        self.ctxs, self.encs, self.mel_len = list(ctxs), list(encs), mel_len
        self.from_pcm, self.post, self.resident, self.read_back = from_pcm, post, resident, read_back
        self.host = [host_windows(s) for s in range(len(self.ctxs))] if resident is None else None
        self.uploads, self.batches, self.outs, self.results, self.pending = [], [], [], [], []
        for s, ctx in enumerate(self.ctxs):
            if resident is not None:
                x = self._forward(s, resident[s])
                res = ctx.pinnedArray(x.rows * x.cols) if read_back else None
                ctx.freeTensor(x)
                u, mels = None, resident[s]
            else:
                m0 = self._upload(s)
                x = self._forward(s, m0)  # once eagerly: weight repacks and pool growth stay out of the recordings
                res = ctx.pinnedArray(x.rows * x.cols) if read_back else None
                ctx.freeTensor(x)
                for m in (m0 if isinstance(m0, list) else [m0]):
                    ctx.freeTensor(m)
                u, mels = ctx.recordBatch(lambda s=s: self._upload(s))
            b, x = ctx.recordBatch(lambda s=s, mels=mels: self._forward(s, mels))
            self.uploads.append(u)
            self.batches.append(b)
            self.outs.append(x)
            self.results.append(res)
        self.next = 0
        self.last = None  # the slot whose forward was enqueued last

    def _upload(self, s):
        """The slot's copies and, from PCM, the log-mel front end: small thread blocks that are not ordered against the
        other slot's forward and fill the SMs its launches leave idle."""
        ctx = self.ctxs[s]
        h = ctx.pushArena()
        if isinstance(self.host[s], np.ndarray):  # one page-locked array holding all windows of the slot back to back
            mels = ctx.upload(self.host[s], self.host[s].size // self.mel_len, self.mel_len)
        else:
            mels = [ctx.upload(m, 1, self.mel_len) for m in self.host[s]]
        if self.from_pcm:
            if isinstance(mels, list):
                mels = ctx.concatRows(mels) if len(mels) > 1 else mels[0]
            mels = ctx.logMelWindows(mels, self.encs[s]["cfg"]["melBins"])
        for m in (mels if isinstance(mels, list) else [mels]):
            ctx.pin(m)
        ctx.popArena(h)
        return mels

    def _forward(self, s, mels):
        ctx = self.ctxs[s]
        h = ctx.pushArena()
        x, _ = encode_batch(ctx, self.encs[s], mels)
        if self.post is not None:
            x = self.post(s, x)
        ctx.pin(x)
        ctx.popArena(h)
        return x

    def _launch(self, s):
        """Enqueue slot s: its copies, then its forward behind the forward enqueued last, then the read-back."""
        ctx = self.ctxs[s]
        if self.uploads[s] is not None:
            self.uploads[s].launch()
        if self.last is not None and self.last != s:
            ctx.waitMark(self.ctxs[self.last])  # this forward starts when the one before it has finished
        self.batches[s].launch()
        ctx.mark()
        self.last = s
        if self.read_back:
            ctx.downloadAsync(self.outs[s], self.results[s])

    def submit(self):
        s = self.next
        self.next = (s + 1) % len(self.ctxs)
        self._launch(s)
        self.pending.append(s)
        if len(self.pending) >= len(self.ctxs):
            return self._read(self.pending.pop(0))
        return None

    def _read(self, s):
        self.ctxs[s].sync()
        return self.results[s]

    def flush(self):
        res = [self._read(s).copy() for s in self.pending]
        self.pending = []
        return res

    def free(self):
        for b in self.batches + self.uploads:
            if b is not None:
                b.free()
