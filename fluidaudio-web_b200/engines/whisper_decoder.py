"""Whisper-style KV-cached decoder, op for op the sequence of
src/engines/asr-whisper/raw-whisper-decoder.js (loadWhisperDecoder :14-72, whisperCrossKV :76-84,
whisperDecodeInit :92-100, whisperDecodeNext :103-142), written only against ComputeContext members.
The reference hard-codes whisper-base sizes (:7-11); here every size is read off the weight shapes so
the same code runs the large-v3-turbo shape (4 layers, D 1280, 20 heads of 64, FFN 5120, vocab 51866).

Each layer: pre-LN causal self-attention against the cache -> pre-LN cross-attention to the encoder
-> pre-LN erf-GELU FFN.  Final LN, logits tied to the token embedding.  q and its bias carry 1/sqrt(HD)
from load time.

Two drivers share the weights:
  * decode_next         one stream, one token: the reference's exact op sequence (M = 1 products);
  * decode_next_streams S streams in lock step: every weight is streamed once per step for all
    streams (M = S products).  Cross-attention is the windowed form of bmmQK / bmmPV (W = S, one
    window per stream).  The growing self-attention caches are laid out time-major,
    [position, stream*D], so that rowsView still selects the filled prefix and the per-stream
    attention is the SAME member with H = S*NH "heads"; the only member outside the reference
    interface is reshapeView (a JS engine re-labels {rows, cols} for that).
Both produce the same logits row for a stream; the tests hold them to the CPU reference's token ids.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np

f32 = np.float32


def infer_config(man: Dict[str, np.ndarray]) -> dict:
    layers = sum(1 for k in man if k.startswith("L") and k.endswith("_sqw"))
    D = man["L0_sqw"].shape[0]
    return dict(D=D, FFN=man["L0_f1w"].shape[1], layers=layers, VOCAB=man["embed"].shape[0], maxPos=man["pos"].shape[0])


def quantize_cols_int8(a: np.ndarray):
    """Symmetric per-output-column int8 of a [K, N] matrix: (q int8 [K,N], scale f32 [N])."""
    scale = (np.abs(a).max(0) / 127.0).astype(f32)
    scale[scale == 0] = 1
    q = np.clip(np.rint(a / scale), -127, 127).astype(np.int8)
    return q, scale


class _W:
    """One weight matrix in whichever storage the variant uses."""

    def __init__(self, ctx, a: np.ndarray, quant: Optional[str]):
        K, N = a.shape
        self.K, self.N, self.quant = K, N, quant
        if quant == "int8":
            q, s = quantize_cols_int8(a)
            self.q = ctx.uploadBytes(np.ascontiguousarray(q).view(np.uint8).reshape(-1))
            self.s = ctx.upload(s, 1, N)
        else:
            self.t = ctx.uploadF16(np.ascontiguousarray(a, dtype=f32), K, N)


def _mm(ctx, x, w: _W, bias=None, act="none"):
    if w.quant == "int8":
        return ctx.matmulInt8(x, w.q, w.s, w.N, w.K, bias=bias, act=act)
    return ctx.matmul(x, w.t, dict(bias=bias, act=act))


def _mm_add(ctx, res, x, w: _W, bias=None):
    """res + (x @ w + bias): the residual rides the product's epilogue where the member takes `add`
    (matmul, compute.d.ts:155); same f32 sum as a separate add()."""
    if w.quant == "int8":
        return ctx.add(res, ctx.matmulInt8(x, w.q, w.s, w.N, w.K, bias=bias))
    return ctx.matmul(x, w.t, dict(bias=bias, add=res))


def load_decoder(ctx, weights: Dict[str, np.ndarray], NH: int, quant: Optional[str] = None) -> dict:
    """raw-whisper-decoder.js:14-72.  quant=None: matrices as f16 storage (the reference's variant);
    quant="int8": matrices as per-column int8 for matmulInt8 (the int8 weight variant)."""
    cfg = infer_config(weights)
    D = cfg["D"]
    HD = D // NH
    cfg.update(NH=NH, HD=HD)
    SCALE = f32(1.0 / math.sqrt(HD))

    def mat(k, s=None):
        a = weights[k].astype(f32)
        if s is not None:
            a = (a * s).astype(f32)
        return _W(ctx, a, quant)

    def vec(k, s=None):
        a = weights[k].astype(f32).reshape(-1)
        if s is not None:
            a = (a * s).astype(f32)
        return ctx.upload(a, 1, a.size)

    layers = []
    for L in range(cfg["layers"]):
        t = lambda s: f"L{L}_{s}"
        layers.append(dict(
            sqw=mat(t("sqw"), SCALE), sqb=vec(t("sqb"), SCALE), skw=mat(t("skw")), svw=mat(t("svw")), svb=vec(t("svb")),
            sow=mat(t("sow")), sob=vec(t("sob")), cqw=mat(t("cqw"), SCALE), cqb=vec(t("cqb"), SCALE), ckw=mat(t("ckw")),
            cvw=mat(t("cvw")), cvb=vec(t("cvb")), cow=mat(t("cow")), cob=vec(t("cob")),
            ln1=(vec(t("ln1w")), vec(t("ln1b"))), ln2=(vec(t("ln2w")), vec(t("ln2b"))), ln3=(vec(t("ln3w")), vec(t("ln3b"))),
            f1w=mat(t("f1w")), f1b=vec(t("f1b")), f2w=mat(t("f2w")), f2b=vec(t("f2b"))))
    # tied vocabulary projection: embed^T [D, VOCABP], vocabulary padded to a multiple of 4 with zero
    # columns (:62-70); consumers slice back to VOCAB so a pad logit of 0.0 never reaches the argmax.
    embed = np.ascontiguousarray(weights["embed"], dtype=f32)
    VOCAB = cfg["VOCAB"]
    VOCABP = (VOCAB + 3) // 4 * 4
    embedTP = np.zeros((D, VOCABP), f32)
    embedTP[:, :VOCAB] = embed.T
    cfg["VOCABP"] = VOCABP
    return dict(layers=layers, embed=embed, embedT=_W(ctx, embedTP, quant), pos=np.ascontiguousarray(weights["pos"], dtype=f32),
                lnf=(vec("lnf_w"), vec("lnf_b")), cfg=cfg)


# ---------------------------------------------------------------------------- one stream (reference form)

def cross_kv(ctx, dec, enc):
    """Per-layer cross-attention K/V from the encoder output, once per clip, pinned (:76-84)."""
    out = []
    for w in dec["layers"]:
        k = _mm(ctx, enc, w["ckw"])
        v = _mm(ctx, enc, w["cvw"], bias=w["cvb"])
        ctx.pin(k)
        ctx.pin(v)
        out.append(dict(k=k, v=v))
    return out


def decode_init(ctx, dec, maxLen: int = 448) -> dict:
    D = dec["cfg"]["D"]
    return dict(n=0, maxLen=maxLen, selfK=[ctx.pin(ctx.alloc(maxLen, D)) for _ in dec["layers"]],
                selfV=[ctx.pin(ctx.alloc(maxLen, D)) for _ in dec["layers"]])


def decode_next(ctx, dec, kv, st, token: int) -> np.ndarray:
    """Feed one token through the cached decoder; logits [VOCAB] for it (:103-142)."""
    cfg = dec["cfg"]
    D, NH, HD, VOCAB = cfg["D"], cfg["NH"], cfg["HD"], cfg["VOCAB"]
    ln = lambda x, lp: ctx.layernorm(x, lp[0], lp[1])
    n = st["n"]
    emb = dec["embed"][token] + dec["pos"][n]
    x = ctx.upload(emb, 1, D)
    arena = ctx.pushArena()

    def body():
        nonlocal x
        for li, w in enumerate(dec["layers"]):
            h = ln(x, w["ln1"])
            q = _mm(ctx, h, w["sqw"], bias=w["sqb"])
            ctx.copyRows(st["selfK"][li], _mm(ctx, h, w["skw"]), n)
            ctx.copyRows(st["selfV"][li], _mm(ctx, h, w["svw"], bias=w["svb"]), n)
            K = ctx.rowsView(st["selfK"][li], n + 1)
            V = ctx.rowsView(st["selfV"][li], n + 1)
            probs = ctx.softmax(ctx.bmmQK(q, K, None, NH, HD))  # [NH, n+1]; only past+current exist -> no mask
            x = ctx.add(x, _mm(ctx, ctx.bmmPV(probs, V, NH, HD), w["sow"], bias=w["sob"]))
            h = ln(x, w["ln2"])
            cq = _mm(ctx, h, w["cqw"], bias=w["cqb"])
            cprobs = ctx.softmax(ctx.bmmQK(cq, kv[li]["k"], None, NH, HD))  # [NH, Tenc]
            x = ctx.add(x, _mm(ctx, ctx.bmmPV(cprobs, kv[li]["v"], NH, HD), w["cow"], bias=w["cob"]))
            h = ln(x, w["ln3"])
            x = ctx.add(x, _mm(ctx, _mm(ctx, h, w["f1w"], bias=w["f1b"], act="gelu_erf"), w["f2w"], bias=w["f2b"]))
        st["n"] = n + 1
        logits = _mm(ctx, ln(x, dec["lnf"]), dec["embedT"])  # [1, VOCABP]
        return ctx.stageDownload(logits)

    try:
        staged = ctx.withBatchSync(body)
        full = staged.read()
        return full[:VOCAB] if full.size > VOCAB else full
    finally:
        ctx.popArena(arena)


def greedy_decode(ctx, dec, enc, prefix: Sequence[int], n_tokens: int, margins: Optional[list] = None) -> List[int]:
    """Forced prefix, then argmax tokens until n_tokens have been produced (no suppress list, no EOT stop:
    the throughput workload's fixed-length form of src/engines/asr-whisper/index.ts:80-97)."""
    kv = cross_kv(ctx, dec, enc)
    st = decode_init(ctx, dec, len(prefix) + n_tokens)
    logits = None
    for t in prefix:
        logits = decode_next(ctx, dec, kv, st, int(t))
    out = []
    for _ in range(n_tokens):
        tok = int(np.argmax(logits))  # first maximum, like the host loop
        if margins is not None:
            top2 = np.partition(logits, -2)[-2:]
            margins.append(float(top2[1] - top2[0]))
        out.append(tok)
        if len(out) < n_tokens:
            logits = decode_next(ctx, dec, kv, st, tok)
    return out


# ---------------------------------------------------------------------------- S streams in lock step

def cross_kv_streams(ctx, dec, encs) -> list:
    """Cross K/V of S clips in ONE product per matrix: the clips' encoder outputs stacked along rows,
    [S*Tenc, D] (a list of [Tenc, D] tensors is concatenated), give k, v [S*Tenc, D] - which is the
    windowed operand layout of bmmQK / bmmPV with W = S."""
    enc_all = ctx.concatRows(list(encs)) if isinstance(encs, (list, tuple)) else encs
    out = []
    for w in dec["layers"]:
        k = ctx.pin(_mm(ctx, enc_all, w["ckw"]))
        v = ctx.pin(_mm(ctx, enc_all, w["cvw"], bias=w["cvb"]))
        out.append(dict(k=k, v=v))
    return out


def decode_init_streams(ctx, dec, S: int, maxLen: int = 448) -> dict:
    D = dec["cfg"]["D"]
    return dict(n=0, S=S, maxLen=maxLen, selfK=[ctx.pin(ctx.alloc(maxLen, S * D)) for _ in dec["layers"]],
                selfV=[ctx.pin(ctx.alloc(maxLen, S * D)) for _ in dec["layers"]])


def step_streams(ctx, dec, kv, st, x, n: int):
    """The device part of one lock-step token for S streams: x [S, D] (embedding + position n) ->
    logits [S, VOCABP].  Same per-row arithmetic as decode_next."""
    cfg = dec["cfg"]
    D, NH, HD = cfg["D"], cfg["NH"], cfg["HD"]
    S = st["S"]
    ln = lambda x, lp: ctx.layernorm(x, lp[0], lp[1])
    for li, w in enumerate(dec["layers"]):
        h = ln(x, w["ln1"])
        q = _mm(ctx, h, w["sqw"], bias=w["sqb"])
        ctx.copyRows(st["selfK"][li], ctx.reshapeView(_mm(ctx, h, w["skw"]), 1, S * D), n)
        ctx.copyRows(st["selfV"][li], ctx.reshapeView(_mm(ctx, h, w["svw"], bias=w["svb"]), 1, S * D), n)
        K = ctx.rowsView(st["selfK"][li], n + 1)
        V = ctx.rowsView(st["selfV"][li], n + 1)
        probs = ctx.softmax(ctx.bmmQK(ctx.reshapeView(q, 1, S * D), K, None, S * NH, HD))  # [S*NH, n+1]
        att = ctx.reshapeView(ctx.bmmPV(probs, V, S * NH, HD), S, D)
        x = _mm_add(ctx, x, att, w["sow"], bias=w["sob"])
        h = ln(x, w["ln2"])
        cq = _mm(ctx, h, w["cqw"], bias=w["cqb"])
        cprobs = ctx.softmax(ctx.bmmQK(cq, kv[li]["k"], None, NH, HD, S))  # one window per stream: [S*NH, Tenc]
        x = _mm_add(ctx, x, ctx.bmmPV(cprobs, kv[li]["v"], NH, HD, S), w["cow"], bias=w["cob"])
        h = ln(x, w["ln3"])
        x = _mm_add(ctx, x, _mm(ctx, h, w["f1w"], bias=w["f1b"], act="gelu_erf"), w["f2w"], bias=w["f2b"])
    return _mm(ctx, ln(x, dec["lnf"]), dec["embedT"])


def decode_next_streams(ctx, dec, kv, st, tokens: Sequence[int], want_logits: bool = False):
    """One token per stream.  Returns (next token ids [S] by first-maximum argmax over the VOCAB real
    columns, logits [S, VOCAB] or None).  The token pick runs on the device when the backend has
    argmaxRowsIndex (8 bytes per stream come back instead of a logits row), else on the host."""
    cfg = dec["cfg"]
    D, VOCAB = cfg["D"], cfg["VOCAB"]
    S, n = st["S"], st["n"]
    emb = dec["embed"][np.asarray(tokens, dtype=np.int64)] + dec["pos"][n][None, :]
    x = ctx.upload(np.ascontiguousarray(emb, dtype=f32), S, D)
    arena = ctx.pushArena()
    on_device = hasattr(ctx, "argmaxRowsIndex") and not want_logits

    def body():
        logits = step_streams(ctx, dec, kv, st, x, n)
        st["n"] = n + 1
        if on_device:
            return ctx.stageDownload(ctx.argmaxRowsIndex(logits, VOCAB))
        return ctx.stageDownload(logits)

    try:
        staged = ctx.withBatchSync(body)
        full = staged.read()
        if on_device:
            return full.reshape(S, 2)[:, 0].astype(np.int64), None
        lg = full.reshape(S, -1)[:, :VOCAB]
        return np.argmax(lg, axis=1).astype(np.int64), lg
    finally:
        ctx.popArena(arena)


def greedy_decode_streams(ctx, dec, encs: Sequence, prefix: Sequence[int], n_tokens: int,
                          kv=None, st=None) -> np.ndarray:
    """S clips decoded in lock step: the forced prefix, then n_tokens greedy tokens per stream.
    Returns int64 [S, n_tokens]."""
    S = len(encs)
    kv = kv if kv is not None else cross_kv_streams(ctx, dec, encs)
    st = st if st is not None else decode_init_streams(ctx, dec, S, len(prefix) + n_tokens)
    st["n"] = 0
    nxt = None
    for t in prefix:
        nxt, _ = decode_next_streams(ctx, dec, kv, st, [int(t)] * S)
    out = np.empty((S, n_tokens), np.int64)
    for i in range(n_tokens):
        out[:, i] = nxt
        if i + 1 < n_tokens:
            nxt, _ = decode_next_streams(ctx, dec, kv, st, nxt)
    return out


# ---------------------------------------------------------------------------- device-resident greedy loop

def resident_tables(ctx, dec) -> dict:
    """The embedding and position tables as device tensors (the reference keeps them on the host and
    gathers there, :66-71); needed only by greedy_decode_streams_resident."""
    if "embedDev" not in dec:
        cfg = dec["cfg"]
        dec["embedDev"] = ctx.pin(ctx.upload(dec["embed"], cfg["VOCAB"], cfg["D"]))
        dec["posDev"] = ctx.pin(ctx.upload(dec["pos"], cfg["maxPos"], cfg["D"]))
    return dec


def greedy_decode_streams_resident(ctx, dec, enc_all, S: int, prefix_idx: Sequence, n_tokens: int, st=None):
    """The whole lock-step greedy decode enqueued with no host round trip: token pick (argmaxRowsIndex)
    and the next token's embedding gather (embedRows) stay on the device, so the sequence of all
    len(prefix)+n_tokens-1 steps can also be recorded once and replayed.  `prefix_idx` holds one device
    tensor [S,1] of token ids per forced prefix position.  Returns the device tensor [n_tokens, S] of
    token ids (as floats).  Needs the backend's optional members; same arithmetic as
    decode_next_streams."""
    cfg = dec["cfg"]
    VOCAB = cfg["VOCAB"]
    resident_tables(ctx, dec)
    kv = cross_kv_streams(ctx, dec, enc_all)
    st = st if st is not None else decode_init_streams(ctx, dec, S, len(prefix_idx) + n_tokens)
    hist = ctx.alloc(n_tokens, S)
    arena = ctx.pushArena()
    try:
        pick = None
        n = 0
        for idx in prefix_idx:
            step = ctx.pushArena()
            x = ctx.embedRows(dec["embedDev"], dec["posDev"], idx, n)
            pick = ctx.argmaxRowsIndex(step_streams(ctx, dec, kv, st, x, n), VOCAB)
            ctx.pin(pick, True)
            ctx.popArena(step)
            n += 1
        for i in range(n_tokens):
            ctx.copyRows(hist, ctx.reshapeView(ctx.sliceCols(pick, 0, 1), 1, S), i)
            if i + 1 == n_tokens:
                break
            step = ctx.pushArena()
            x = ctx.embedRows(dec["embedDev"], dec["posDev"], pick, n)
            pick = ctx.argmaxRowsIndex(step_streams(ctx, dec, kv, st, x, n), VOCAB)
            ctx.pin(pick, True)
            ctx.popArena(step)
            n += 1
    finally:
        ctx.popArena(arena)
        for c in kv:
            ctx.freeTensor(c["k"])
            ctx.freeTensor(c["v"])
    st["n"] = n
    return hist
