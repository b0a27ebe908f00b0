"""Parity of the CUDA hot path with the CPU oracle, through the C ABI (CudaContext -> libfa_cuda.so).

Tolerances are the reference's own (scripts/backend-conformance.mjs:67-141: 1e-3 for f32/int8/int4
small cases, 2e-2 for the f16-B route, 5e-2 all-f16) and the stated bars for the large shapes:
int32 accumulators bit-exact; int8 outputs within 1e-3 relative; f16/int4 within 2e-2 max-abs on
unit-scale outputs.
"""
import os

import numpy as np
import pytest

from oracle.wasm_oracle import T, WasmOracle, int8_gemm_i32

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "conformance_gemm.npz"))


def rel_err(got, ref):
    """max |got-ref| relative to max(|ref|, rms(ref)) elementwise: 'within 1e-3 relative' without
    blowing up on outputs that happen to be near zero."""
    ref = ref.astype(np.float64)
    rms = np.sqrt((ref ** 2).mean()) + 1e-30
    return float((np.abs(got - ref) / np.maximum(np.abs(ref), rms)).max())


def gin(name, key):
    return GOLD[f"{name}.in.{key}"]


# ---- the reference gate's seeded cases (fixtures hold inputs and the oracle's outputs) ----------

@pytest.mark.parametrize("act", ["none", "gelu", "gelu_erf", "tanh", "relu", "silu"])
def test_conformance_matmul_bias_act(ctx, act):
    name = f"matmul_bias_{act}"
    a, b, bias = gin(name, "a"), gin(name, "b"), gin(name, "bias")
    out = ctx.download(ctx.matmul(ctx.upload(a, 37, 53), ctx.upload(b, 53, 41), bias=ctx.upload(bias, 1, 41), act=act))
    assert np.abs(out.reshape(37, 41) - GOLD[name]).max() <= 1e-3


def test_conformance_matmul_relu_add(ctx):
    name = "matmul_relu_add"
    a, b, d = gin(name, "a"), gin(name, "b"), gin(name, "add")
    out = ctx.download(ctx.matmul(ctx.upload(a, 64, 128), ctx.upload(b, 128, 256), {"act": "relu", "add": ctx.upload(d, 64, 256)}))
    assert np.abs(out.reshape(64, 256) - GOLD[name]).max() <= 1e-3


def test_conformance_variants(ctx):
    a, b = gin("matmulV2_gelu", "a"), gin("matmulV2_gelu", "b")
    out = ctx.download(ctx.matmulV2(ctx.upload(a, 33, 48), ctx.upload(b, 48, 52), act="gelu"))
    assert np.abs(out.reshape(33, 52) - GOLD["matmulV2_gelu"]).max() <= 1e-3
    a, b = gin("matmulV3", "a"), gin("matmulV3", "b")
    out = ctx.download(ctx.matmulV3(ctx.upload(a, 33, 64), ctx.upload(b, 64, 48)))
    assert np.abs(out.reshape(33, 48) - GOLD["matmulV3"]).max() <= 1e-3
    a, b, bias = (gin("matmulV4_bias_silu", k) for k in ("a", "b", "bias"))
    out = ctx.download(ctx.matmulV4(ctx.upload(a, 129, 64), ctx.upload(b, 64, 132), bias=ctx.upload(bias, 1, 132), act="silu"))
    assert np.abs(out.reshape(129, 132) - GOLD["matmulV4_bias_silu"]).max() <= 1e-3


def test_conformance_f16_routes(ctx):
    a, b = gin("matmulF16", "a"), gin("matmulF16", "b")
    out = ctx.downloadF16(ctx.matmulF16(ctx.uploadF16(a, 40, 64), ctx.uploadF16(b, 64, 64)))
    assert np.abs(out.reshape(40, 64) - GOLD["matmulF16"]).max() <= 5e-2
    name = "matmul_f16B_bias_silu"
    a, b, bias = gin(name, "a"), gin(name, "b"), gin(name, "bias")
    out = ctx.download(ctx.matmul(ctx.upload(a, 65, 128), ctx.uploadF16(b, 128, 256), bias=ctx.upload(bias, 1, 256), act="silu"))
    assert np.abs(out.reshape(65, 256) - GOLD[name]).max() <= 2e-2


def test_conformance_int8_and_int4(ctx):
    name = "matmulInt8_bias_relu"
    a, wq, s, bias = (gin(name, k) for k in ("a", "wq", "scale", "bias"))
    out = ctx.download(ctx.matmulInt8(ctx.upload(a, 9, 20), ctx.uploadBytes(wq), ctx.upload(s, 1, 16), 16, 20,
                                      {"bias": ctx.upload(bias, 1, 16), "act": "relu"}))
    assert np.abs(out.reshape(9, 16) - GOLD[name]).max() <= 1e-3
    name = "matmulNBits"
    a, bq, zp, s = (gin(name, k) for k in ("a", "bq", "zp", "scales"))
    out = ctx.download(ctx.matmulNBits(ctx.upload(a, 7, 64), ctx.uploadBytes(bq), ctx.upload(s, 1, 16), ctx.uploadBytes(zp), 8))
    assert np.abs(out.reshape(7, 8) - GOLD[name]).max() <= 1e-3


# ---- int8: tensor-core route ---------------------------------------------------------------------

def _int8_case(rng, M, K, N):
    a = rng.standard_normal((M, K)).astype(np.float32)
    wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    sc = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
    return a, wq, sc


@pytest.mark.parametrize("M,K,N", [(128, 512, 256), (512, 1024, 4096), (200, 328, 136), (16, 1024, 512), (1, 2048, 384)])
@pytest.mark.parametrize("limbs", [2, 3])
def test_int8_tensor_core_vs_oracle(ctx, M, K, N, limbs):
    rng = np.random.default_rng(0)
    a, wq, sc = _int8_case(rng, M, K, N)
    bias = rng.standard_normal(N).astype(np.float32)
    ctx.setOption("int8_limbs", limbs)
    try:
        y = ctx.download(ctx.matmulInt8(ctx.upload(a, M, K), ctx.uploadBytes(wq), ctx.upload(sc, 1, N), N, K,
                                        bias=ctx.upload(bias, 1, N), act="none")).reshape(M, N)
    finally:
        ctx.setOption("int8_limbs", 2)
    ora = WasmOracle(threads=True)
    ref = ora.matmulInt8(T(a, M, K), ora.uploadBytes(wq), T(sc, 1, N), N, K, bias=T(bias, 1, N), loop_order="ikj").array()
    assert rel_err(y, ref) <= 1e-3


@pytest.mark.parametrize("M,K,N", [(128, 512, 256), (512, 1024, 4096), (77, 200, 136)])
def test_int8_int32_accumulators_bit_exact(ctx, M, K, N):
    rng = np.random.default_rng(1)
    aq = rng.integers(-127, 128, (M, K), dtype=np.int8)
    wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    got = ctx.int8GemmI32(aq, ctx.uploadBytes(wq), N, K)
    assert np.array_equal(got, int8_gemm_i32(aq, wq))


def test_int8_w8a8_mode_matches_oracle_on_quantised_operands(ctx):
    """One limb = plain per-row int8 activation quantisation: fp32 outputs equal the oracle run on
    the same quantised operands (dequantised activations), to f32 rounding."""
    rng = np.random.default_rng(2)
    M, K, N = 256, 1024, 512
    a, wq, sc = _int8_case(rng, M, K, N)
    ctx.setOption("int8_limbs", 1)
    try:
        y = ctx.download(ctx.matmulInt8(ctx.upload(a, M, K), ctx.uploadBytes(wq), ctx.upload(sc, 1, N), N, K)).reshape(M, N)
    finally:
        ctx.setOption("int8_limbs", 2)
    a_scale = (np.abs(a).max(axis=1) / np.float32(127)).astype(np.float32)
    aq = np.clip(np.rint(a / a_scale[:, None]), -127, 127).astype(np.int8)
    acc = int8_gemm_i32(aq, wq)
    ref = acc.astype(np.float32) * a_scale[:, None] * sc[None, :]
    assert rel_err(y, ref) <= 1e-5


# ---- f16-weight GEMM -----------------------------------------------------------------------------

@pytest.mark.parametrize("M,K,N", [(256, 1024, 1024), (300, 520, 264), (1024, 1024, 3072), (4, 1024, 1024)])
def test_f16_weight_gemm_vs_oracle(ctx, M, K, N):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    add = rng.standard_normal((M, N)).astype(np.float32)
    y = ctx.download(ctx.matmul(ctx.upload(a, M, K), ctx.uploadF16(w, K, N), bias=ctx.upload(bias, 1, N), act="silu",
                                add=ctx.upload(add, M, N))).reshape(M, N)
    ora = WasmOracle(threads=True)
    ref = ora.matmul(T(a, M, K), T(w, K, N), bias=T(bias, 1, N), act="silu", add=T(add, M, N)).array()
    assert np.abs(y - ref).max() <= 2e-2


# ---- int4 ---------------------------------------------------------------------------------------

def _int4_case(rng, M, K, N, signed_zp=True):
    nblk = -(-K // 32)
    zpb = -(-nblk // 2)
    bq = rng.integers(0, 256, N * nblk * 16, dtype=np.uint8)
    scales = rng.uniform(5e-3, 2e-2, N * nblk).astype(np.float16).astype(np.float32)
    zp = np.full(N * zpb, 0x88, np.uint8) if signed_zp else rng.integers(0, 256, N * zpb, dtype=np.uint8)
    a = rng.standard_normal((M, K)).astype(np.float16).astype(np.float32)
    return a, bq, scales, zp


@pytest.mark.parametrize("M", [1, 4, 16])
@pytest.mark.parametrize("N", [2048, 8192])
def test_int4_decode_shapes_vs_oracle(ctx, M, N):
    K = 2048
    rng = np.random.default_rng(1)
    a, bq, scales, zp = _int4_case(rng, M, K, N)
    y = ctx.download(ctx.matmulNBits(ctx.upload(a, M, K), ctx.uploadBytes(bq), ctx.upload(scales, 1, scales.size),
                                     ctx.uploadBytes(zp), N)).reshape(M, N)
    ora = WasmOracle(threads=True)
    ref = ora.matmulNBits(T(a, M, K), ora.uploadBytes(bq), T(scales, 1, scales.size), ora.uploadBytes(zp), N).array()
    assert np.abs(y - ref).max() <= 2e-2


def test_int4_partial_block_and_random_zero_points(ctx):
    rng = np.random.default_rng(5)
    for (M, K, N) in [(8, 100, 64), (40, 1000, 328), (130, 4352, 1024)]:
        a, bq, scales, zp = _int4_case(rng, M, K, N, signed_zp=False)
        y = ctx.download(ctx.matmulNBits(ctx.upload(a, M, K), ctx.uploadBytes(bq), ctx.upload(scales, 1, scales.size),
                                         ctx.uploadBytes(zp), N)).reshape(M, N)
        ora = WasmOracle(threads=True)
        ref = ora.matmulNBits(T(a, M, K), ora.uploadBytes(bq), T(scales, 1, scales.size), ora.uploadBytes(zp), N).array()
        assert np.abs(y - ref).max() <= 2e-2, (M, K, N)


MMA_CASES = [(5, 2048, 2048, 64), (8, 100, 64, 64), (16, 2048, 8192, 64), (13, 1000, 328, 64), (16, 4352, 1024, 0),
             (2, 2048, 2048, 64), (16, 64, 8, 64)]


@pytest.mark.parametrize("M,K,N,hilo_rows", MMA_CASES, ids=[f"{c[0]}x{c[1]}x{c[2]}-{c[3]}" for c in MMA_CASES])
def test_int4_few_rows_streamed_nibbles_mma(ctx, M, K, N, hilo_rows):
    """int4 products with up to 16 activation rows stream the 4-bit weights once and multiply with mma.sync
    (option "nbits_mma_rows"): partial last block, unsigned random zero-points, more than 64 blocks per row (a warp
    then walks two quads), with and without the residue plane of the activations - against the oracle, and against
    the tensor-core GEMM on the dequantised copy (option off)."""
    rng = np.random.default_rng(M * 7 + N)
    a, bq, scales, zp = _int4_case(rng, M, K, N, signed_zp=False)
    a = (a + rng.standard_normal(a.shape).astype(np.float32) * 1e-3).astype(np.float32)  # not f16-representable
    ora = WasmOracle(threads=True)
    ref = ora.matmulNBits(T(a, M, K), ora.uploadBytes(bq), T(scales, 1, scales.size), ora.uploadBytes(zp), N).array()
    ctx.setOption("f16_hilo_rows", hilo_rows)
    outs = []
    try:
        for rows in (17, 0):  # 17: this kernel whatever N is (by default only while a thread block walks few column groups)
            ctx.setOption("nbits_mma_rows", rows)
            ctx.setOption("gemv_rows", 0 if M <= 4 else 4)  # route the few-row cases here, not to the dp4a GEMV
            h = ctx.pushArena()
            y = ctx.download(ctx.matmulNBits(ctx.upload(a, M, K), ctx.uploadBytes(bq), ctx.upload(scales, 1, scales.size),
                                             ctx.uploadBytes(zp), N)).reshape(M, N)
            ctx.popArena(h)
            outs.append(y)
    finally:
        ctx.setOption("nbits_mma_rows", 16)
        ctx.setOption("gemv_rows", 4)
        ctx.setOption("f16_hilo_rows", 64)
    assert np.abs(outs[0] - ref).max() <= 2e-2, float(np.abs(outs[0] - ref).max())
    assert np.abs(outs[0] - outs[1]).max() <= 2e-2


# ---- size-independent properties at full size ------------------------------------------------------

def test_int8_full_size_linearity_and_exactness(ctx):
    """The int8 benchmark shape (512x1024x4096): y(a1+a2) = y(a1)+y(a2) holds exactly for the int32
    accumulators, and zero activations give exactly the bias."""
    rng = np.random.default_rng(0)
    M, K, N = 512, 1024, 4096
    wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    wb = ctx.uploadBytes(wq)
    a1 = rng.integers(-60, 61, (M, K), dtype=np.int8)
    a2 = rng.integers(-60, 61, (M, K), dtype=np.int8)
    y1, y2, y12 = (ctx.int8GemmI32(x, wb, N, K) for x in (a1, a2, (a1 + a2).astype(np.int8)))
    assert np.array_equal(y1 + y2, y12)
    sc = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    z = ctx.download(ctx.matmulInt8(ctx.upload(np.zeros((M, K), np.float32), M, K), wb, ctx.upload(sc, 1, N), N, K,
                                    bias=ctx.upload(bias, 1, N))).reshape(M, N)
    assert np.array_equal(z, np.broadcast_to(bias, (M, N)))


# ---- decode-size products on the CUDA-core GEMV kernels (M <= 4) ---------------------------------------

@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("K,N", [(2048, 8192), (2048, 2048), (96, 200), (4096, 333)])
def test_gemv_nbits_matches_oracle(ctx, oracle, M, K, N):
    rng = np.random.default_rng(M * 7 + N)
    nblk = K // 32
    a = rng.standard_normal((M, K)).astype(np.float32)
    bq = rng.integers(0, 256, N * nblk * 16, dtype=np.uint8)
    scales = rng.uniform(5e-3, 2e-2, N * nblk).astype(np.float32)
    zp = rng.integers(0, 256, N * ((nblk + 1) // 2), dtype=np.uint8)
    ref = oracle.matmulNBits(oracle.upload(a, M, K), oracle.uploadBytes(bq), oracle.upload(scales, 1, scales.size),
                             oracle.uploadBytes(zp), N).array()
    ctx.startProfile(64)
    got = ctx.download(ctx.matmulNBits(ctx.upload(a, M, K), ctx.uploadBytes(bq), ctx.upload(scales, 1, scales.size),
                                       ctx.uploadBytes(zp), N)).reshape(M, N)
    labels = [e["label"] for e in ctx.endProfile()]
    assert "gemv_nbits" in labels and not any(l.startswith(("tc_gemm", "gemm_simt", "nbits_simt")) for l in labels), labels
    # two int8 digits of the row maximum: error bound 2^-15 * max|a| * sum|w| per output; outputs are O(sqrt(K)*0.06)
    assert np.abs(got - ref).max() <= 2e-3 * max(1.0, float(np.abs(ref).max()) / 3.0)
    assert np.abs(got - ref).max() <= 2e-2


@pytest.mark.parametrize("M", [1])
@pytest.mark.parametrize("K,N", [(1280, 1280), (1280, 5120), (5120, 1280), (1280, 51868), (77, 260), (4100, 64)])
def test_gemv_f16_weights_matches_oracle(ctx, oracle, M, K, N):
    rng = np.random.default_rng(M + K + N)
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    add = rng.standard_normal((M, N)).astype(np.float32)
    ref = oracle.matmul(oracle.upload(a, M, K), oracle.upload(b, K, N),
                        dict(bias=oracle.upload(bias, 1, N), act="gelu_erf", add=oracle.upload(add, M, N))).array()
    ctx.startProfile(64)
    got = ctx.download(ctx.matmul(ctx.upload(a, M, K), ctx.uploadF16(b, K, N),
                                  dict(bias=ctx.upload(bias, 1, N), act="gelu_erf", add=ctx.upload(add, M, N))))
    labels = [e["label"] for e in ctx.endProfile()]
    assert "gemv_f16" in labels and not any(l.startswith(("tc_gemm", "gemm_simt", "nbits_simt")) for l in labels), labels
    assert np.abs(got.reshape(M, N) - ref).max() <= 2e-5  # f32 activations, f32 accumulation: only summation order differs


@pytest.mark.parametrize("M", [1])
@pytest.mark.parametrize("K,N", [(1024, 4096), (1280, 51872), (333, 64), (5120, 1280)])
def test_gemv_int8_weights_matches_oracle(ctx, oracle, M, K, N):
    rng = np.random.default_rng(M + K + N)
    a = rng.standard_normal((M, K)).astype(np.float32)
    wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    sc = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    ref = oracle.matmulInt8(oracle.upload(a, M, K), oracle.uploadBytes(wq.view(np.uint8).reshape(-1)), oracle.upload(sc, 1, N),
                            N, K, bias=oracle.upload(bias, 1, N), act="relu").array()
    ctx.startProfile(64)
    got = ctx.download(ctx.matmulInt8(ctx.upload(a, M, K), ctx.uploadBytes(wq.view(np.uint8).reshape(-1)), ctx.upload(sc, 1, N),
                                      N, K, bias=ctx.upload(bias, 1, N), act="relu"))
    labels = [e["label"] for e in ctx.endProfile()]
    assert "gemv_i8" in labels and not any(l.startswith(("tc_gemm", "gemm_simt", "nbits_simt")) for l in labels), labels
    assert np.abs(got.reshape(M, N) - ref).max() <= 1e-3 * max(1.0, float(np.abs(ref).max()))
    assert np.abs(got.reshape(M, N) - ref).max() <= 5e-5 * max(1.0, float(np.abs(ref).max()))


def test_gemv_option_off_uses_tensor_cores(ctx, oracle):
    rng = np.random.default_rng(1)
    M, K, N = 1, 1280, 1280
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
    ref = oracle.matmul(oracle.upload(a, M, K), oracle.upload(b, K, N)).array()
    ctx.setOption("gemv_rows", 0)
    try:
        ctx.startProfile(64)
        got = ctx.download(ctx.matmul(ctx.upload(a, M, K), ctx.uploadF16(b, K, N)))
        assert "tc_gemm_f16" in [e["label"] for e in ctx.endProfile()]
    finally:
        ctx.setOption("gemv_rows", 4)
    assert np.abs(got.reshape(M, N) - ref).max() <= 2e-5


@pytest.mark.parametrize("M,K,N", [(16, 2048, 8192), (8, 2048, 2048), (130, 1056, 300), (5, 96, 4100)])
def test_int4_unpack_in_shared_memory_variant(ctx, oracle, M, K, N):
    """The tensor-core int4 kernel that streams 4-bit tiles and unpacks them in shared memory (option
    nbits_fused): same product as the oracle within the int4 tolerance, ragged N and odd block counts too."""
    rng = np.random.default_rng(M + K + N)
    nblk = K // 32
    a = rng.standard_normal((M, K)).astype(np.float32)
    bq = rng.integers(0, 256, N * nblk * 16, dtype=np.uint8)
    scales = rng.uniform(5e-3, 2e-2, N * nblk).astype(np.float32)
    zp = rng.integers(0, 256, N * ((nblk + 1) // 2), dtype=np.uint8)
    ref = oracle.matmulNBits(oracle.upload(a, M, K), oracle.uploadBytes(bq), oracle.upload(scales, 1, scales.size),
                             oracle.uploadBytes(zp), N).array()
    ctx.setOption("nbits_fused", 1)
    try:
        ctx.startProfile(64)
        got = ctx.download(ctx.matmulNBits(ctx.upload(a, M, K), ctx.uploadBytes(bq), ctx.upload(scales, 1, scales.size),
                                           ctx.uploadBytes(zp), N)).reshape(M, N)
        labels = [e["label"] for e in ctx.endProfile()]
    finally:
        ctx.setOption("nbits_fused", 0)
    assert "tc_gemm_nbits" in labels, labels
    assert np.abs(got - ref).max() <= 2e-2 * max(1.0, float(np.abs(ref).max()) / 3.0)


def test_matmul_scatter_writes_every_result_buffer(ctx, oracle):
    """The product whose epilogue stores its column block into several [M, ldc] result buffers (the fused
    all-gather of the N-sharded sweep), here with three buffers on one GPU."""
    rng = np.random.default_rng(12)
    M, K, Ns, ldc, col0 = 300, 256, 192, 640, 256
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, Ns)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
    bias = rng.standard_normal(Ns).astype(np.float32)
    ref = oracle.matmul(oracle.upload(a, M, K), oracle.upload(b, K, Ns), dict(bias=oracle.upload(bias, 1, Ns), act="relu")).array()
    fill = np.full((M, ldc), -7.0, np.float32)
    bufs = [ctx.upload(fill, M, ldc) for _ in range(3)]
    ctx.matmulScatter(ctx.upload(a, M, K), ctx.uploadF16(b, K, Ns), [ctx.devicePtr(t) for t in bufs], ldc, col0,
                      bias=ctx.upload(bias, 1, Ns), act="relu")
    first = None
    for t in bufs:
        got = ctx.download(t).reshape(M, ldc)
        assert np.all(got[:, :col0] == -7.0) and np.all(got[:, col0 + Ns:] == -7.0)  # only the block is written
        assert np.abs(got[:, col0:col0 + Ns] - ref).max() <= 2e-2
        first = got if first is None else first
        assert np.array_equal(got, first)  # every buffer holds the same bits


def test_matmul_scatter_single_buffer_wide_pitch_few_rows(ctx, oracle):
    """One result buffer whose row pitch is wider than the product, with 65..128 rows and few column tiles: the
    shape class that would otherwise take the K-split cluster form, whose finish writes rows at pitch N."""
    rng = np.random.default_rng(13)
    M, K, Ns, ldc, col0 = 96, 1024, 256, 640, 130  # col0 not a multiple of 4 either
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, Ns)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
    ref = oracle.matmul(oracle.upload(a, M, K), oracle.upload(b, K, Ns)).array()
    buf = ctx.upload(np.full((M, ldc), -7.0, np.float32), M, ldc)
    ctx.matmulScatter(ctx.upload(a, M, K), ctx.uploadF16(b, K, Ns), [ctx.devicePtr(buf)], ldc, col0)
    got = ctx.download(buf).reshape(M, ldc)
    assert np.all(got[:, :col0] == -7.0) and np.all(got[:, col0 + Ns:] == -7.0)
    assert np.abs(got[:, col0:col0 + Ns] - ref).max() <= 2e-2


def test_hidden_layer_result_is_lazy_and_consistent(ctx, oracle):
    """A product with a fused activation writes only the packed f16 operand of the next product; its f32
    storage is filled (f16-rounded) when something else reads it.  The chained product is bit-identical with
    the option off, and a direct read stays within the f16-route tolerance of the oracle."""
    rng = np.random.default_rng(21)
    M, K, N, N2 = 300, 256, 512, 192
    a = rng.standard_normal((M, K)).astype(np.float32)
    w1 = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
    w2 = (rng.standard_normal((N, N2)) / np.sqrt(N)).astype(np.float16).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    ref_h = oracle.matmul(oracle.upload(a, M, K), oracle.upload(w1, K, N), dict(bias=oracle.upload(bias, 1, N), act="silu")).array()
    outs = {}
    for lazy in (1, 0):
        ctx.setOption("lazy_f32", lazy)
        try:
            A, W1, W2, B = ctx.upload(a, M, K), ctx.uploadF16(w1, K, N), ctx.uploadF16(w2, N, N2), ctx.upload(bias, 1, N)
            ctx.startProfile(64)
            h = ctx.matmul(A, W1, dict(bias=B, act="silu"))
            y = ctx.download(ctx.matmul(h, W2)).reshape(M, N2)
            labels_chain = [e["label"] for e in ctx.endProfile()]
            ctx.startProfile(64)
            hd = ctx.download(h).reshape(M, N)
            labels_read = [e["label"] for e in ctx.endProfile()]
            outs[lazy] = (y, hd, labels_chain, labels_read)
        finally:
            ctx.setOption("lazy_f32", 1)
    y1, h1, chain1, read1 = outs[1]
    y0, h0, chain0, read0 = outs[0]
    assert np.array_equal(y1, y0)                      # the next product sees the same f16 operand either way
    assert "unpack_a_f16" not in chain1 and "unpack_a_f16" in read1 and "unpack_a_f16" not in read0
    assert np.array_equal(h1, h0.astype(np.float16).astype(np.float32))  # the lazy copy is the f16 rounding of the f32 one
    assert np.abs(h1 - ref_h).max() <= 2e-2
    # reading through other members works too: a view and an elementwise op on a fresh lazy result
    A, W1, B = ctx.upload(a, M, K), ctx.uploadF16(w1, K, N), ctx.upload(bias, 1, N)
    h = ctx.matmul(A, W1, dict(bias=B, act="silu"))
    v = ctx.download(ctx.rowsView(h, 7)).reshape(7, N)
    assert np.array_equal(v, h1[:7])
    h = ctx.matmul(A, W1, dict(bias=B, act="silu"))
    s2 = ctx.download(ctx.scale(h, 2.0)).reshape(M, N)
    assert np.array_equal(s2, h1 * 2.0)


# ---- f32-storage B: tensor-core route (value + residue planes on kind::tf32) -------------------------------

@pytest.mark.parametrize("M,K,N,opts", [(512, 1024, 4096, {}), (256, 256, 256, dict(bias=True, act="gelu_erf")),
                                        (300, 520, 264, dict(bias=True, act="silu", add=True)), (1024, 4096, 1024, dict(add=True))])
def test_f32_weight_gemm_on_tensor_cores_vs_oracle(ctx, M, K, N, opts):
    """f32 x f32 at the sizes the reference routes to its fastest f32 kernel (M, N, K >= 256,
    src/gpu/compute.js:426; its own check of that kernel is scripts/gemm-verify-v4.mjs:22-50 at 2e-4).  The
    gate's 1e-3 holds with orders of magnitude to spare because both operands keep ~20 bits."""
    rng = np.random.default_rng(31)
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32) if opts.get("bias") else None
    add = rng.standard_normal((M, N)).astype(np.float32) if opts.get("add") else None
    act = opts.get("act", "none")
    ctx.startProfile(16)
    got = ctx.download(ctx.matmul(ctx.upload(a, M, K), ctx.upload(b, K, N), bias=ctx.upload(bias, 1, N) if bias is not None else None,
                                  act=act, add=ctx.upload(add, M, N) if add is not None else None)).reshape(M, N)
    labels = {e["label"] for e in ctx.endProfile()}
    assert "tc_gemm_tf32x3" in labels, labels  # the tensor-core route ran, not the CUDA-core kernel
    rows = np.unique(np.concatenate([[0, M - 1], rng.integers(0, M, 48)]))
    ora = WasmOracle(threads=True)
    ref = ora.matmul(T(a[rows], len(rows), K), T(b, K, N), bias=T(bias, 1, N) if bias is not None else None, act=act,
                     add=T(add[rows], len(rows), N) if add is not None else None).array()
    assert np.abs(got[rows] - ref).max() <= 2e-4
    assert rel_err(got[rows], ref) <= 1e-3


def test_f32_weight_small_shapes_stay_exact_f32(ctx):
    """300 x 64 x 300 (K below the threshold): the any-shape f32 kernel, as before."""
    rng = np.random.default_rng(32)
    M, K, N = 300, 64, 300
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    got = ctx.download(ctx.matmul(ctx.upload(a, M, K), ctx.upload(b, K, N))).reshape(M, N)
    ora = WasmOracle(threads=True)
    assert np.abs(got - ora.matmul(T(a, M, K), T(b, K, N)).array()).max() <= 1e-4


# ---- int8 weights resident on the device, f16 activations (matmulInt8Operand) ----------------------------

@pytest.mark.parametrize("M,K,N,opts", [(300, 520, 264, dict(bias=True, act="silu")), (512, 1024, 4096, {}),
                                        (1024, 4096, 1024, dict(bias=True, add=True)), (200, 256, 192, dict(operandOnly=True)),
                                        (6016, 1024, 3072, dict(bias=True, operandOnly=True)), (16, 1024, 512, dict(bias=True, add=True))])
def test_int8_resident_weights_f16_activations_vs_oracle(ctx, M, K, N, opts):
    """Against the oracle's matmulInt8 (f32 activations): the f16 rounding of the activations is the only difference,
    so the f16-B route's tolerance applies (2e-2 on unit-scale outputs)."""
    rng = np.random.default_rng(41)
    a = rng.standard_normal((M, K)).astype(np.float32)
    wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    sc = (rng.uniform(0.5, 1.5, N) / (73.0 * np.sqrt(K))).astype(np.float32)  # unit-scale outputs
    bias = rng.standard_normal(N).astype(np.float32) if opts.get("bias") else None
    add = rng.standard_normal((M, N)).astype(np.float32) if opts.get("add") else None
    act = opts.get("act", "none")
    o = dict(act=act, operandOnly=bool(opts.get("operandOnly")))
    if bias is not None:
        o["bias"] = ctx.upload(bias, 1, N)
    if add is not None:
        o["add"] = ctx.upload(add, M, N)
    h = ctx.pushArena()
    try:
        ctx.startProfile(16)
        got = ctx.download(ctx.matmulInt8Operand(ctx.upload(a, M, K), ctx.uploadBytes(wq), ctx.upload(sc, 1, N), N, K, o)).reshape(M, N)
        labels = {e["label"] for e in ctx.endProfile()}
    finally:
        ctx.popArena(h)
    if M > 64:
        assert "tc_gemm_i8w_f16a" in labels, labels
    rows = np.unique(np.concatenate([[0, M - 1], rng.integers(0, M, 48)]))
    ora = WasmOracle(threads=True)
    ref = ora.matmulInt8(T(a[rows], len(rows), K), ora.uploadBytes(wq), T(sc, 1, N), N, K, bias=T(bias, 1, N) if bias is not None else None,
                         act=act).array()
    if add is not None:
        ref = ref + add[rows]
    assert np.abs(got[rows] - ref).max() <= 2e-2


# ---- CTA pairs (tcgen05 cta_group::2) ---------------------------------------------------------------

PAIR_CASES = [
    (1200, 256, 512, dict()),                                    # 8 x 5 tiles: barely more tiles than SMs
    (2500, 320, 1024, dict(bias=True)),                          # ragged M (last tile 196 of 224 rows), ragged K chunk
    (3000, 1024, 768, dict(bias=True, act="silu", operand_only=True)),  # f16 operand out only
    (2111, 512, 1280, dict(bias=True, add=True)),                # residual read, odd row count
    (6016, 1024, 1024, dict(add=True)),                          # the encoder's residual products at their real size
    (2050, 192, 768, dict(bias=True, add=True, act="silu")),     # residual behind an activation, two rows in the last block
    (19001, 64, 256, dict(bias=True)),                           # one K chunk per tile, one column pair, ragged last tile
    (4097, 96, 512, dict(act="relu")),                           # K not a multiple of the 64-element chunk
]


@pytest.mark.parametrize("M,K,N,kw", PAIR_CASES, ids=[f"{c[0]}x{c[1]}x{c[2]}" for c in PAIR_CASES])
def test_pair_kernel_matches_one_cta_kernel_and_oracle(ctx, M, K, N, kw):
    """Products with more tiles than SMs run on pairs of thread blocks sharing one 256-lane MMA (option "tc_pair",
    default on).  The pair kernel accumulates the same K chunks in the same order into the same accumulators as the
    one-block kernel, so the two must agree bit for bit; a sample of rows is also checked against the oracle.  A
    residual operand reaches the epilogue through the copy engine (option "tc_tma_add", default on) or by plain loads:
    the same additions in the same order, bit for bit as well."""
    rng = np.random.default_rng(M + N)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float16).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32) if kw.get("bias") else None
    r = rng.standard_normal((M, N)).astype(np.float32) if kw.get("add") else None
    outs = []
    try:
        # pairs, one-block kernel, pairs with per-lane stores, pairs with the residual read by plain loads
        for pair, tma_store, tma_add in ((1, 1, 1), (0, 1, 1), (1, 0, 1), (1, 1, 0)):
            ctx.setOption("tc_pair", pair)
            ctx.setOption("tc_tma_store", tma_store)
            ctx.setOption("tc_tma_add", tma_add)
            h = ctx.pushArena()
            try:
                opts = dict(act=kw.get("act", "none"))
                if b is not None:
                    opts["bias"] = ctx.upload(b, 1, N)
                if r is not None:
                    opts["add"] = ctx.upload(r, M, N)
                if kw.get("operand_only"):
                    opts["operandOnly"] = True
                wt = ctx.uploadF16(w, K, N)
                outs.append(ctx.download(ctx.matmul(ctx.upload(a, M, K), wt, opts)).reshape(M, N).copy())
                ctx.freeTensor(wt)
            finally:
                ctx.popArena(h)
    finally:
        ctx.setOption("tc_pair", 1)
        ctx.setOption("tc_tma_store", 1)
        ctx.setOption("tc_tma_add", 1)
    assert np.array_equal(outs[0], outs[1])
    assert np.array_equal(outs[0], outs[2])
    assert np.array_equal(outs[0], outs[3])
    rows = np.unique(np.concatenate([[0, 1, M - 2, M - 1], rng.integers(0, M, 28)]))
    ora = WasmOracle(threads=True)
    ref = ora.matmul(T(a[rows], len(rows), K), T(w, K, N), bias=T(b, 1, N) if b is not None else None, act=kw.get("act", "none"),
                     add=T(r[rows], len(rows), N) if r is not None else None).array()
    assert float(np.abs(outs[0][rows] - ref).max()) <= 2e-2
