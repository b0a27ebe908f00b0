"""Glue ops (what the encoder/decoder forwards call between GEMMs) against the CPU oracle, through the
C ABI.  Tolerances follow scripts/backend-conformance.mjs (1e-4 for normalisation/elementwise, 1e-3 for
the attention products and convolutions)."""
import numpy as np
import pytest

from oracle.wasm_oracle import T, WasmOracle

pytestmark = pytest.mark.gpu

ORA = WasmOracle()


def up(ctx, a):
    a = np.ascontiguousarray(a, np.float32)
    r, c = (1, a.size) if a.ndim == 1 else a.shape
    return ctx.upload(a, r, c), T(a, r, c)


def close(ctx, got, ref, tol):
    g = ctx.download(got).reshape(ref.rows, ref.cols)
    assert (got.rows, got.cols) == (ref.rows, ref.cols)
    assert np.abs(g - ref.array()).max() <= tol


def test_layernorm_softmax(ctx):
    rng = np.random.default_rng(0)
    for R, C in [(7, 33), (64, 1024), (3, 1500)]:
        x, xo = up(ctx, rng.standard_normal((R, C)) * 3)
        g, go = up(ctx, rng.standard_normal(C))
        b, bo = up(ctx, rng.standard_normal(C))
        close(ctx, ctx.layernorm(x, g, b), ORA.layernorm(xo, go, bo), 1e-4)
        close(ctx, ctx.softmax(x), ORA.softmax(xo), 1e-5)


def test_layernorm_operand_is_the_f16_operand_of_the_same_layernorm(ctx):
    """layernormOperand (optional member): identical to layernorm for few rows; for many rows the tensor is the
    product's packed f16 operand (read-back = f16 rounding of layernorm's result) and a product of it equals the
    product of the plain layernorm bit for bit, eagerly and when replayed from a recording."""
    rng = np.random.default_rng(12)
    for R, C in [(7, 64), (200, 1024), (130, 320), (90, 1500), (100, 64)]:
        x, xo = up(ctx, rng.standard_normal((R, C)) * 3)
        g, go = up(ctx, rng.standard_normal(C))
        b, bo = up(ctx, rng.standard_normal(C))
        plain = ctx.download(ctx.layernorm(x, g, b))
        got = ctx.download(ctx.layernormOperand(x, g, b))
        if R <= 64 or C > 1024 or C % 64 or R * C < 32768:  # too small for a sure tensor-core consumer: plain layernorm
            assert np.array_equal(got, plain)
        else:
            assert np.array_equal(got, plain.astype(np.float16).astype(np.float32))
    R, C, N = 200, 1024, 256
    x, _ = up(ctx, rng.standard_normal((R, C)))
    g, _ = up(ctx, rng.standard_normal(C))
    b, _ = up(ctx, rng.standard_normal(C))
    w = ctx.uploadF16((rng.standard_normal((C, N)) * 0.05).astype(np.float32), C, N)
    want = ctx.download(ctx.matmul(ctx.layernorm(x, g, b), w))
    assert np.array_equal(ctx.download(ctx.matmul(ctx.layernormOperand(x, g, b), w)), want)

    host = ctx.pinnedArray(R * C)
    host[:] = rng.standard_normal(R * C).astype(np.float32)

    def body():
        h = ctx.layernormOperand(ctx.upload(host, R, C), g, b)
        return ctx.matmul(h, w), h

    body()
    batch, (y, h) = ctx.recordBatch(body)
    for _ in range(2):
        host[:] = rng.standard_normal(R * C).astype(np.float32)
        batch.launch()
        ln = ctx.layernorm(ctx.upload(host, R, C), g, b)
        assert np.array_equal(ctx.download(y), ctx.download(ctx.matmul(ln, w)))
        assert np.array_equal(ctx.download(h), ctx.download(ln).astype(np.float16).astype(np.float32))
    batch.free()


def test_layernorm_chain_equals_the_two_calls(ctx):
    rng = np.random.default_rng(13)
    for R, C in [(200, 1024), (130, 320), (9, 64), (70, 1500)]:
        x, _ = up(ctx, rng.standard_normal((R, C)) * 2)
        g1, _ = up(ctx, rng.standard_normal(C))
        b1, _ = up(ctx, rng.standard_normal(C))
        g2, _ = up(ctx, rng.standard_normal(C))
        b2, _ = up(ctx, rng.standard_normal(C))
        y, z = ctx.layernormChain(x, g1, b1, g2, b2)
        y0 = ctx.layernorm(x, g1, b1)
        z0 = ctx.layernormOperand(y0, g2, b2)
        assert np.array_equal(ctx.download(y), ctx.download(y0))
        assert np.array_equal(ctx.download(z), ctx.download(z0))


def test_elementwise_and_movement(ctx):
    rng = np.random.default_rng(1)
    a, ao = up(ctx, rng.standard_normal((37, 50)))
    b, bo = up(ctx, rng.standard_normal((37, 50)))
    r, ro = up(ctx, rng.standard_normal(50))
    close(ctx, ctx.add(a, b), ORA.add(ao, bo), 0)
    close(ctx, ctx.mul(a, r), ORA.mul(ao, ro), 0)  # row broadcast
    close(ctx, ctx.scale(a, 0.37), ORA.scale(ao, 0.37), 1e-6)
    close(ctx, ctx.silu(a), ORA.silu(ao), 1e-5)
    close(ctx, ctx.relu(a), ORA.relu(ao), 0)
    close(ctx, ctx.transpose(a), ORA.transpose(ao), 0)
    close(ctx, ctx.sliceCols(a, 7, 20), ORA.sliceCols(ao, 7, 20), 0)
    close(ctx, ctx.sliceRows(a, 5, 9), ORA.sliceRows(ao, 5, 9), 0)
    g, go = up(ctx, rng.standard_normal((64, 41)))
    close(ctx, ctx.glu(g), ORA.glu(go), 1e-5)
    d, do = up(ctx, np.zeros((37, 80)))
    close(ctx, ctx.setCols(d, a, 11), ORA.setCols(do, ao, 11), 0)
    c1, c1o = up(ctx, rng.standard_normal((3, 9)))
    c2, c2o = up(ctx, rng.standard_normal((5, 9)))
    close(ctx, ctx.concatRows([c1, c2]), ORA.concatRows([c1o, c2o]), 0)
    dst, dsto = up(ctx, np.zeros((10, 9)))
    close(ctx, ctx.copyRows(dst, c2, 4), ORA.copyRows(dsto, c2o, 4), 0)
    s, so = up(ctx, rng.standard_normal((6, 4 * 5)))
    close(ctx, ctx.subReshape(s, 6, 4, 5), ORA.subReshape(so, 6, 4, 5), 0)


def test_attention_products_and_rel_shift(ctx):
    rng = np.random.default_rng(2)
    W, H, HD, Tq = 3, 4, 32, 19
    q, qo = up(ctx, rng.standard_normal((W * Tq, H * HD)))
    k, ko = up(ctx, rng.standard_normal((W * Tq, H * HD)))
    pb, pbo = up(ctx, rng.standard_normal(H * HD))
    pos, poso = up(ctx, rng.standard_normal((2 * Tq - 1, H * HD)))
    ac, aco = ctx.bmmQK(q, k, pb, H, HD, W), ORA.bmmQK(qo, ko, pbo, H, HD, W)
    close(ctx, ac, aco, 1e-3)
    bd, bdo = ctx.bmmQK(q, pos, None, H, HD, W, True), ORA.bmmQK(qo, poso, None, H, HD, W, True)
    close(ctx, bd, bdo, 1e-3)
    sh, sho = ctx.relShiftB(bd, W * H), ORA.relShiftB(bdo, W * H)
    close(ctx, sh, sho, 1e-3)
    p, po = ctx.softmax(ctx.add(ac, sh)), ORA.softmax(ORA.add(aco, sho))
    close(ctx, ctx.bmmPV(p, k, H, HD, W), ORA.bmmPV(po, ko, H, HD, W), 1e-3)


def test_attention_products_full_head_size_tensor_core_route(ctx):
    """Parakeet head geometry (8 heads of 128, 188 frames): the batched tcgen05 route, f16 operands."""
    rng = np.random.default_rng(5)
    W, H, HD, Tq = 3, 8, 128, 188
    q, qo = up(ctx, rng.standard_normal((W * Tq, H * HD)) * 0.3)
    k, ko = up(ctx, rng.standard_normal((W * Tq, H * HD)) * 0.3)
    pb, pbo = up(ctx, rng.standard_normal(H * HD) * 0.02)
    pos, poso = up(ctx, rng.standard_normal((2 * Tq - 1, H * HD)) * 0.3)
    ac, aco = ctx.bmmQK(q, k, pb, H, HD, W), ORA.bmmQK(qo, ko, pbo, H, HD, W)
    close(ctx, ac, aco, 2e-2)
    bd, bdo = ctx.bmmQK(q, pos, None, H, HD, W, True), ORA.bmmQK(qo, poso, None, H, HD, W, True)
    close(ctx, bd, bdo, 2e-2)
    po = ORA.softmax(ORA.add(aco, ORA.relShiftB(bdo, W * H)))
    p = ctx.upload(po.array(), po.rows, po.cols)
    close(ctx, ctx.bmmPV(p, k, H, HD, W), ORA.bmmPV(po, ko, H, HD, W), 2e-3)


def test_convolutions(ctx):
    rng = np.random.default_rng(3)
    # depthwise conv over time with fused silu (the conformer conv module)
    Cc, L, k = 48, 77, 9
    x, xo = up(ctx, rng.standard_normal((Cc, L)))
    w, wo = up(ctx, rng.standard_normal(Cc * k))
    b, bo = up(ctx, rng.standard_normal(Cc))
    close(ctx, ctx.conv1d(x, w, cout=Cc, k=k, groups=Cc, padLeft=4, padRight=4, bias=b, act="silu"),
          ORA.conv1d(xo, wo, cout=Cc, k=k, groups=Cc, padLeft=4, padRight=4, bias=bo, act="silu"), 1e-4)
    # subsampling convs: cin=1 3x3 s2, depthwise 3x3 s2, pointwise
    h, wd, C0 = 41, 24, 16
    img, imgo = up(ctx, rng.standard_normal((1, h * wd)))
    w0, w0o = up(ctx, rng.standard_normal(C0 * 9))
    b0, b0o = up(ctx, rng.standard_normal(C0))
    o = dict(cout=C0, cin=1, h=h, w=wd, kh=3, kw=3, strideH=2, strideW=2, padTop=1, padBottom=1, padLeft=1, padRight=1, act="relu")
    y = ctx.conv2d(img, w0, dict(o, bias=b0))
    yo = ORA.conv2d(imgo, w0o, C0, 1, h, wd, 3, 3, bias=b0o, strideH=2, strideW=2, padTop=1, padBottom=1, padLeft=1, padRight=1, act="relu")
    close(ctx, y, yo, 1e-4)
    h2, w2 = (h + 2 - 3) // 2 + 1, (wd + 2 - 3) // 2 + 1
    wd_, wdo = up(ctx, rng.standard_normal(C0 * 9))
    y2 = ctx.conv2d(y, wd_, cout=C0, cin=C0, h=h2, w=w2, kh=3, kw=3, strideH=2, strideW=2, padTop=1, padBottom=1, padLeft=1, padRight=1, groups=C0)
    y2o = ORA.conv2d(yo, wdo, C0, C0, h2, w2, 3, 3, strideH=2, strideW=2, padTop=1, padBottom=1, padLeft=1, padRight=1, groups=C0)
    close(ctx, y2, y2o, 1e-4)
    h3, w3 = (h2 + 2 - 3) // 2 + 1, (w2 + 2 - 3) // 2 + 1
    wp, wpo = up(ctx, rng.standard_normal(C0 * C0))
    close(ctx, ctx.conv2d(y2, wp, cout=C0, cin=C0, h=h3, w=w3, kh=1, kw=1, act="relu"),
          ORA.conv2d(y2o, wpo, C0, C0, h3, w3, 1, 1, act="relu"), 1e-4)


def test_argmax_rows(ctx):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((5, 51868)).astype(np.float32)
    x[2, 100] = x[2, 40000] = 50.0  # tie -> lowest index
    out = ctx.download(ctx.argmaxRowsIndex(ctx.upload(x, 5, 51868))).reshape(5, 2)
    assert np.array_equal(out[:, 0].astype(np.int64), x.argmax(axis=1))
    assert np.array_equal(out[:, 1], x.max(axis=1))
    x[:, 51866:] = 99.0  # pad columns beyond the limit never win
    out = ctx.download(ctx.argmaxRowsIndex(ctx.upload(x, 5, 51868), 51866)).reshape(5, 2)
    assert np.array_equal(out[:, 0].astype(np.int64), x[:, :51866].argmax(axis=1))


def test_conv_module_fast_members_match_the_op_sequence(ctx):
    """conv1dWindows and gluDwConvTimeMajor (optional members) against the reference's per-window sequence
    transpose -> glu -> sliceCols/conv1d/setCols -> transpose run on the oracle."""
    rng = np.random.default_rng(6)
    W, T, D, k = 3, 37, 512, 9
    pre1, pre1o = up(ctx, rng.standard_normal((W * T, 2 * D)))
    dw, dwo_ = up(ctx, rng.standard_normal(D * k) * 0.3)
    b, bo = up(ctx, rng.standard_normal(D) * 0.1)
    opts = dict(cout=D, k=k, groups=D, padLeft=4, padRight=4, act="silu")
    gluo = ORA.glu(ORA.transpose(pre1o))
    ref = ORA.alloc(D, W * T)
    for wi in range(W):
        ORA.setCols(ref, ORA.conv1d(ORA.sliceCols(gluo, wi * T, T), dwo_, dict(opts, bias=bo)), wi * T)
    glu = ctx.glu(ctx.transpose(pre1))
    close(ctx, ctx.conv1dWindows(glu, dw, dict(opts, bias=b), W), ref, 1e-4)
    # when large enough that its consumer is a tensor-core product, the fused member keeps its result as that product's f16 operand alone: the f32
    # read-back is that operand (f16 rounding of the exact result); with lazy_f32 off it stores the f32 result
    lazy = ctx.gluDwConvTimeMajor(pre1, dw, dict(opts, bias=b), W)
    ctx.setOption("lazy_f32", 0)
    try:
        exact = ctx.gluDwConvTimeMajor(pre1, dw, dict(opts, bias=b), W)
    finally:
        ctx.setOption("lazy_f32", 1)
    close(ctx, exact, ORA.transpose(ref), 1e-4)
    e = ctx.download(exact)
    assert np.array_equal(ctx.download(lazy), e.astype(np.float16).astype(np.float32))


def test_unshard_cols_matches_host_statement(ctx, pkg):
    from fluidaudio_web_b200 import sharding

    rng = np.random.default_rng(8)
    for world, M, ns in ((2, 5, 8), (4, 33, 12), (8, 16, 128), (1, 3, 4)):
        g = rng.standard_normal((world * M, ns)).astype(np.float32)
        got = ctx.download(ctx.unshardCols(ctx.upload(g, world * M, ns), world)).reshape(M, world * ns)
        assert np.array_equal(got, sharding.unshard_cols_host(g, world))


@pytest.mark.parametrize("geom", [
    dict(cout=16, cin=1, kh=3, kw=3, strideH=2, strideW=2, padTop=1, padBottom=1, padLeft=1, padRight=1, groups=1, act="relu"),
    dict(cout=16, cin=16, kh=3, kw=3, strideH=2, strideW=2, padTop=1, padBottom=1, padLeft=1, padRight=1, groups=16, act="none"),
    dict(cout=64, cin=64, kh=1, kw=1, groups=1, act="relu"),   # pointwise -> tensor cores, batched over windows
    dict(cout=8, cin=4, kh=3, kw=2, strideH=1, strideW=2, padTop=0, padBottom=1, padLeft=1, padRight=0, groups=2, act="silu"),
])
def test_conv2d_windows_equals_per_window_conv2d(ctx, geom):
    """The window-batched front-end members against the per-window members they replace (bit for bit: same
    kernels, one more grid dimension)."""
    rng = np.random.default_rng(geom["cout"] + geom["cin"])
    W, h, w = 3, 37, 50
    cin, cout, g = geom["cin"], geom["cout"], geom["groups"]
    x = rng.standard_normal((W, cin * h * w)).astype(np.float32)
    wt = rng.standard_normal((cout, (cin // g) * geom["kh"] * geom["kw"])).astype(np.float32)
    b = rng.standard_normal(cout).astype(np.float32)
    wt_t, b_t = ctx.upload(wt, wt.shape[0], wt.shape[1]), ctx.upload(b, 1, cout)
    opts = dict(geom, h=h, w=w, bias=b_t)
    got = ctx.download(ctx.conv2dWindows(ctx.upload(x, W, x.shape[1]), wt_t, opts, W)).reshape(W, -1)
    for i in range(W):
        one = ctx.download(ctx.conv2d(ctx.upload(x[i], 1, x.shape[1]), wt_t, opts))
        assert np.array_equal(got[i], one.reshape(-1)), (geom, i)


def test_sub_reshape_windows(ctx):
    rng = np.random.default_rng(1)
    W, C, Tsub, F = 4, 6, 9, 5
    x = rng.standard_normal((W, C * Tsub * F)).astype(np.float32)
    got = ctx.download(ctx.subReshapeWindows(ctx.upload(x, W, x.shape[1]), C, Tsub, F, W)).reshape(W, Tsub, C * F)
    for i in range(W):
        one = ctx.download(ctx.subReshape(ctx.upload(x[i], C, Tsub * F), C, Tsub, F)).reshape(Tsub, C * F)
        assert np.array_equal(got[i], one)


@pytest.mark.parametrize("W,C,Tsub,F", [(3, 8, 21, 16), (2, 256, 47, 16), (1, 16, 10, 4)])
def test_sub_reshape_vector_form_and_packed_operand(ctx, W, C, Tsub, F):
    """F % 4 == 0 takes the four-column kernel, which also hands the result over as the packed f16 operand of the
    linear layer (and, when large enough, as that alone): values against the host statement of the move, and a
    product of the result against the product of an uploaded copy."""
    rng = np.random.default_rng(C + Tsub)
    x = rng.standard_normal((W, C * Tsub * F)).astype(np.float32)
    want = x.reshape(W, C, Tsub, F).transpose(0, 2, 1, 3).reshape(W * Tsub, C * F)
    xt = ctx.upload(x, W, x.shape[1]) if W > 1 else ctx.upload(x[0], C, Tsub * F)
    got = ctx.subReshapeWindows(xt, C, Tsub, F, W) if W > 1 else ctx.subReshape(xt, C, Tsub, F)
    g = ctx.download(got).reshape(W * Tsub, C * F)
    lazy = W * Tsub > 64 and (C * F) % 64 == 0 and W * Tsub * C * F >= 32768
    assert np.array_equal(g, want.astype(np.float16).astype(np.float32) if lazy else want)
    if (C * F) % 64 == 0:
        wl = ctx.uploadF16((rng.standard_normal((C * F, 128)) * 0.05).astype(np.float32), C * F, 128)
        again = ctx.subReshapeWindows(xt, C, Tsub, F, W) if W > 1 else ctx.subReshape(xt, C, Tsub, F)
        a = ctx.download(ctx.matmul(again, wl))
        b = ctx.download(ctx.matmul(ctx.upload(want, W * Tsub, C * F), wl))
        assert np.abs(a - b).max() <= (0 if W * Tsub > 64 else 2e-3)


@pytest.mark.parametrize("h,Cc,W,bias", [(70, 64, 3, True), (37, 128, 2, True), (131, 64, 1, False), (7, 256, 2, True)])
def test_conv_stem_windows_equals_the_three_layer_sequence(ctx, h, Cc, W, bias):
    """convStemWindows (optional member) against the conv2dWindows calls it replaces, bit for bit, over image
    heights that leave ragged last row groups; and it declines geometries outside its kernel's range."""
    rng = np.random.default_rng(h + Cc)
    w = 128
    x = ctx.upload(rng.standard_normal((W, h * w)).astype(np.float32), W, h * w)
    mk = lambda n, s: ctx.upload((rng.standard_normal(n) * s).astype(np.float32), 1, n)
    layers = [dict(w=mk(Cc * 9, 0.3), b=mk(Cc, 0.1) if bias else None), dict(w=mk(Cc * 9, 0.3), b=mk(Cc, 0.1) if bias else None),
              dict(w=mk(Cc * Cc, 0.1), b=mk(Cc, 0.1) if bias else None)]
    got = ctx.convStemWindows(x, layers, Cc, h, w, W)
    assert got is not None
    geo = [(1, 3, 2, 1, "relu", 1), (Cc, 3, 2, Cc, "none", 1), (Cc, 1, 1, 1, "relu", 0)]
    s, Hh, Wd = x, h, w
    for l, (cin, k, st, gr, act, p) in zip(layers, geo):
        s = ctx.conv2dWindows(s, l["w"], dict(cout=Cc, cin=cin, h=Hh, w=Wd, kh=k, kw=k, bias=l["b"], strideH=st, strideW=st,
                                              padTop=p, padBottom=p, padLeft=p, padRight=p, groups=gr, act=act), W)
        Hh, Wd = (Hh + 2 * p - k) // st + 1, (Wd + 2 * p - k) // st + 1
    assert (got.rows, got.cols) == (W, Cc * Hh * Wd)  # (conv2dWindows of one window is shaped [C, H*W] like conv2d)
    assert np.array_equal(ctx.download(got).reshape(-1), ctx.download(s).reshape(-1))
    x64 = ctx.upload(rng.standard_normal((W, h * 64)).astype(np.float32), W, h * 64)
    assert ctx.convStemWindows(x64, layers, Cc, h, 64, W) is None  # not a 128-column image: declined


@pytest.mark.parametrize("W,H,T", [(3, 8, 188), (2, 2, 100), (1, 3, 192), (2, 1, 16), (1, 2, 57)])
def test_attn_fused_matches_the_op_sequence(ctx, W, H, T):
    """attnFused (optional member) in both of its forms - the one-kernel form and the batched-GEMM form - against
    the reference's op sequence bmmQK x2 -> relShiftB -> add -> softmax -> bmmPV on the oracle; the result must also
    work as the row operand of the projection that follows (it is stored as that operand alone by default)."""
    rng = np.random.default_rng(W * 1000 + T)
    HD, S = 128, H * 128
    q, qo = up(ctx, rng.standard_normal((W * T, S)) * 0.3)
    k, ko = up(ctx, rng.standard_normal((W * T, S)) * 0.3)
    v, vo = up(ctx, rng.standard_normal((W * T, S)) * 0.5)
    pos, poso = up(ctx, rng.standard_normal((2 * T - 1, S)) * 0.3)
    pbu, pbuo = up(ctx, rng.standard_normal(S) * 0.1)
    pbv, pbvo = up(ctx, rng.standard_normal(S) * 0.1)
    aco = ORA.bmmQK(qo, ko, pbuo, H, HD, W)
    bdo = ORA.relShiftB(ORA.bmmQK(qo, poso, pbvo, H, HD, W, True), W * H)
    ref = ORA.bmmPV(ORA.softmax(ORA.add(aco, bdo)), vo, H, HD, W)
    wout = (rng.standard_normal((S, 64)) * 0.05).astype(np.float32)
    for one_kernel in (1, 0):
        ctx.setOption("attn_one_kernel", one_kernel)
        try:
            got = ctx.attnFused(q, k, v, pos, pbu, pbv, H, HD, W)
            if got is None:
                assert one_kernel == 0  # the GEMM form may decline small shapes; the one-kernel form covers T in 16..192
                continue
            y = ctx.download(ctx.matmul(got, ctx.uploadF16(wout, S, 64))).reshape(W * T, 64)
            close(ctx, got, ref, 3e-3)
            assert np.abs(y - ref.array() @ wout.astype(np.float16).astype(np.float32)).max() <= 5e-3
        finally:
            ctx.setOption("attn_one_kernel", 1)
    # the same attention over the columns of one fused projection [q | k | v]: bit-identical to the separate tensors
    one = ctx.attnFused(q, k, v, pos, pbu, pbv, H, HD, W)
    cat = np.concatenate([ctx.download(x).reshape(W * T, S) for x in (q, k, v)], axis=1)
    fused = ctx.attnFusedQKV(ctx.upload(cat, W * T, 3 * S), pos, pbu, pbv, H, HD, W)
    assert fused is not None and np.array_equal(ctx.download(fused), ctx.download(one))
    # ... and over a projection that exists only as its packed f16 operand (matmul with the operandOnly hint)
    if W * T > 64 and W * T * 3 * S * 64 >= (1 << 21):
        xin = rng.standard_normal((W * T, 256)).astype(np.float32)
        wcat = (rng.standard_normal((256, 3 * S)) * 0.02).astype(np.float32)  # unit-scale scores, as in the model
        bcat, _ = up(ctx, rng.standard_normal(3 * S) * 0.1)
        xt, wt = ctx.upload(xin, W * T, 256), ctx.uploadF16(wcat, 256, 3 * S)
        plain = ctx.matmul(xt, wt, dict(bias=bcat))
        hinted = ctx.matmul(xt, wt, dict(bias=bcat, operandOnly=True))
        a = ctx.download(ctx.attnFusedQKV(plain, pos, pbu, pbv, H, HD, W))
        b = ctx.download(ctx.attnFusedQKV(hinted, pos, pbu, pbv, H, HD, W))
        assert np.abs(a - b).max() <= 3e-3 * max(1.0, float(np.abs(a).max()))
        # the operand-only result is the plain result rounded to f16; the two launches may sum K in a different
        # order (a thin product splits K over a cluster), so allow the rounding to land on the neighbouring f16
        pl16 = ctx.download(plain).astype(np.float16).astype(np.float32)
        hd = ctx.download(hinted)
        assert np.abs(hd - pl16).max() <= 2.0 ** -10 * max(1.0, float(np.abs(pl16).max()))
        assert (hd != pl16).mean() < 0.01


@pytest.mark.parametrize("h,Cc,W,bias", [(75, 64, 3, True), (19, 128, 2, True), (70, 64, 1, False), (8, 256, 2, True)])
def test_conv_dw_pw_windows_equals_the_two_layer_sequence(ctx, h, Cc, W, bias):
    """convDwPwWindows (optional member) against the two conv2dWindows calls it replaces, bit for bit."""
    rng = np.random.default_rng(h * 7 + Cc)
    w = 32
    x = ctx.upload(rng.standard_normal((W, Cc * h * w)).astype(np.float32), W, Cc * h * w)
    mk = lambda n, s: ctx.upload((rng.standard_normal(n) * s).astype(np.float32), 1, n)
    layers = [dict(w=mk(Cc * 9, 0.3), b=mk(Cc, 0.1) if bias else None), dict(w=mk(Cc * Cc, 0.1), b=mk(Cc, 0.1) if bias else None)]
    got = ctx.convDwPwWindows(x, layers, Cc, h, w, W)
    assert got is not None
    s, Hh, Wd = x, h, w
    for l, (k, st, gr, act, p) in zip(layers, [(3, 2, Cc, "none", 1), (1, 1, 1, "relu", 0)]):
        s = ctx.conv2dWindows(s, l["w"], dict(cout=Cc, cin=Cc, h=Hh, w=Wd, kh=k, kw=k, bias=l["b"], strideH=st, strideW=st,
                                              padTop=p, padBottom=p, padLeft=p, padRight=p, groups=gr, act=act), W)
        Hh, Wd = (Hh + 2 * p - k) // st + 1, (Wd + 2 * p - k) // st + 1
    assert (got.rows, got.cols) == (W, Cc * Hh * Wd)
    assert np.array_equal(ctx.download(got).reshape(-1), ctx.download(s).reshape(-1))
    x64 = ctx.upload(rng.standard_normal((W, Cc * h * 64)).astype(np.float32), W, Cc * h * 64)
    assert ctx.convDwPwWindows(x64, layers, Cc, h, 64, W) is None  # not a 32-column map: declined
