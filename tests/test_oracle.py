"""Pins the CPU oracle to the known-answer material the reference holds for the path.

The reference has no golden files for its GEMMs.  What it has are (1) in-script
reference formulas with tolerances in scripts/wasm-verify.mjs:27-59,167-228 - restated
here in float64 numpy - and (2) the seeded inputs of scripts/backend-conformance.mjs.
"""
import numpy as np
import pytest

from oracle.wasm_oracle import ACT, LIB, Mulberry32, T, WasmOracle, int8_gemm_i32


def _mulberry32_py(seed, n):
    out = []
    for _ in range(n):
        seed = (seed + 0x6D2B79F5) & 0xFFFFFFFF
        t = ((seed ^ (seed >> 15)) * (1 | seed)) & 0xFFFFFFFF
        t = ((t + (((t ^ (t >> 7)) * (61 | t)) & 0xFFFFFFFF)) & 0xFFFFFFFF) ^ t
        out.append(((t ^ (t >> 14)) & 0xFFFFFFFF) / 4294967296)
    return np.array(out), seed


def test_mulberry32_matches_js_definition():
    ref, _ = _mulberry32_py(0x5EED, 257)
    got = Mulberry32(0x5EED).data(257)
    assert np.array_equal(got, (ref - 0.5).astype(np.float32))
    assert np.array_equal(Mulberry32(0x5EED).bytes(257), np.floor(ref * 256).astype(np.uint8))


def _gelu64(x):
    return 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x**3)))


def test_matmul_bias_gelu_wasm_verify_formula(oracle):
    # scripts/wasm-verify.mjs:27-43: 80x512x300, bias, gelu, tol 1e-3
    rng = np.random.default_rng(11)
    M, K, N = 80, 512, 300
    A, B, bias = (rng.random(s) - 0.5 for s in ((M, K), (K, N), (N,)))
    A, B, bias = A.astype(np.float32), B.astype(np.float32), bias.astype(np.float32)
    ref = _gelu64(A.astype(np.float64) @ B.astype(np.float64) + bias)
    got = oracle.matmul(T(A, M, K), T(B, K, N), bias=T(bias, 1, N), act="gelu").array()
    assert np.abs(got - ref).max() <= 1e-3


def test_matmul_silu_wasm_verify_formula(oracle):
    # scripts/wasm-verify.mjs:44-59
    rng = np.random.default_rng(12)
    M, K, N = 32, 128, 64
    A = (rng.random((M, K)) - 0.5).astype(np.float32)
    B = (rng.random((K, N)) - 0.5).astype(np.float32)
    s = A.astype(np.float64) @ B.astype(np.float64)
    ref = s / (1 + np.exp(-s))
    assert np.abs(oracle.matmul(T(A, M, K), T(B, K, N), act="silu").array() - ref).max() <= 1e-3


def test_matmul_int8_wasm_verify_formula(oracle):
    # scripts/wasm-verify.mjs:167-191: per-column symmetric quantiser, 40x256x128, tol 1e-3
    rng = np.random.default_rng(13)
    M, K, N = 40, 256, 128
    A = (rng.random((M, K)) - 0.5).astype(np.float32)
    W = (rng.random((K, N)) - 0.5).astype(np.float32)
    sc = np.abs(W).max(axis=0) / 127
    sc[sc == 0] = 1
    sc = sc.astype(np.float32)
    q = np.clip(np.floor(W / sc + 0.5), -127, 127).astype(np.int8)  # Math.round = floor(x+0.5)
    ref = (A.astype(np.float64) @ q.astype(np.float64)) * sc
    o = oracle.matmulInt8(T(A, M, K), oracle.uploadBytes(q.view(np.uint8)), T(sc, 1, N), N, K)
    assert np.abs(o.array() - ref).max() <= 1e-3
    # loop-interchanged and threaded forms are bit-identical to the reference loop order
    o2 = oracle.matmulInt8(T(A, M, K), oracle.uploadBytes(q.view(np.uint8)), T(sc, 1, N), N, K, loop_order="ikj")
    assert np.array_equal(o.data, o2.data)
    o3 = WasmOracle(threads=True).matmulInt8(T(A, M, K), oracle.uploadBytes(q.view(np.uint8)), T(sc, 1, N), N, K)
    assert np.array_equal(o.data, o3.data)


def test_matmul_nbits_wasm_verify_formula(oracle):
    # scripts/wasm-verify.mjs:192-228: M=8 N=64 K=100 (partial last block), random bytes
    rng = np.random.default_rng(14)
    M, N, K, blk = 8, 64, 100, 32
    nblk = -(-K // blk)
    zpb = -(-nblk // 2)
    Bq = rng.integers(0, 256, N * nblk * 16, dtype=np.uint8)
    scales = (np.abs(rng.random(N * nblk) - 0.5) * 0.1 + 0.02).astype(np.float32)
    zp = rng.integers(0, 256, N * zpb, dtype=np.uint8)
    A = ((rng.random((M, K)) - 0.5) * 0.1).astype(np.float32)
    nib = np.stack([Bq & 15, Bq >> 4], axis=-1).reshape(N, nblk * 32).astype(np.float64)[:, :K]
    zpn = np.stack([zp & 15, zp >> 4], axis=-1).reshape(N, zpb * 2)[:, :nblk].astype(np.float64)
    w = (nib - np.repeat(zpn, 32, axis=1)[:, :K]) * np.repeat(scales.reshape(N, nblk).astype(np.float64), 32, axis=1)[:, :K]
    ref = A.astype(np.float64) @ w.T
    o = oracle.matmulNBits(T(A, M, K), oracle.uploadBytes(Bq), T(scales, 1, scales.size), oracle.uploadBytes(zp), N)
    assert np.abs(o.array() - ref).max() <= 1e-3
    o2 = WasmOracle(threads=True).matmulNBits(T(A, M, K), oracle.uploadBytes(Bq), T(scales, 1, scales.size), oracle.uploadBytes(zp), N)
    assert np.array_equal(o.data, o2.data)


def test_matmul_f32_is_unfused_k_ordered(oracle):
    # lib.rs:76-91: c = c + a*b with separate roundings, k ascending
    rng = np.random.default_rng(15)
    M, K, N = 5, 37, 9
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    ref = np.zeros((M, N), np.float32)
    for k in range(K):
        ref = (ref + (A[:, k:k + 1] * B[k:k + 1, :]).astype(np.float32)).astype(np.float32)
    assert np.array_equal(oracle.matmul(T(A, M, K), T(B, K, N)).array(), ref)
    assert np.array_equal(WasmOracle(threads=True).matmul(T(A, M, K), T(B, K, N)).array(), ref)


@pytest.mark.parametrize("act", list(ACT))
def test_activation_table(act):
    # wasm-context.js:12-38 / kernels/actf.js:5-22, including the clamps
    xs = np.array([-40.0, -25.0, -3.0, -0.5, 0.0, 0.5, 3.0, 25.0, 40.0])
    got = np.array([LIB.js_apply_act(float(x), ACT[act]) for x in xs])
    if act == "none":
        ref = xs
    elif act == "relu":
        ref = np.maximum(xs, 0)
    elif act == "tanh":
        ref = np.tanh(xs)
    elif act == "silu":
        ref = xs / (1 + np.exp(-np.clip(xs, -30, 30)))
    elif act == "gelu":
        ref = 0.5 * xs * (1 + np.tanh(np.clip(0.7978845608028654 * (xs + 0.044715 * xs**3), -20, 20)))
    else:
        from math import erf
        ref = np.array([0.5 * x * (1 + erf(x / np.sqrt(2))) for x in xs])
        assert np.abs(got - ref).max() < 2e-6  # A&S 7.1.26 approximation error
        return
    assert np.allclose(got, ref, rtol=1e-14, atol=0)


def test_int32_restatement_exact():
    rng = np.random.default_rng(16)
    aq = rng.integers(-127, 128, (7, 96), dtype=np.int8)
    wq = rng.integers(-127, 128, (96, 24), dtype=np.int8)
    assert np.array_equal(int8_gemm_i32(aq, wq), aq.astype(np.int64) @ wq.astype(np.int64))


def test_golden_conformance_cases(oracle):
    """Oracle outputs on the reference gate's seeded GEMM cases match the committed fixtures."""
    import os
    from tests.golden.gen_golden import conformance_gemm_cases

    path = os.path.join(os.path.dirname(__file__), "golden", "conformance_gemm.npz")
    gold = np.load(path)
    for name, _inputs, out in conformance_gemm_cases(oracle):
        assert np.array_equal(gold[name], out), name


def test_glue_ops_against_numpy(oracle):
    rng = np.random.default_rng(17)
    x = rng.standard_normal((7, 33)).astype(np.float32)
    g = rng.standard_normal(33).astype(np.float32)
    b = rng.standard_normal(33).astype(np.float32)
    x64 = x.astype(np.float64)
    ln = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
    assert np.abs(oracle.layernorm(T(x, 7, 33), T(g, 1, 33), T(b, 1, 33)).array() - ln).max() < 1e-5
    e = np.exp(x64 - x64.max(1, keepdims=True))
    assert np.abs(oracle.softmax(T(x, 7, 33)).array() - e / e.sum(1, keepdims=True)).max() < 1e-6
    assert np.array_equal(oracle.transpose(T(x, 7, 33)).array(), x.T)
    # bmmQK / bmmPV with W windows, H heads
    W, H, HD, Tq = 2, 3, 8, 5
    q = rng.standard_normal((W * Tq, H * HD)).astype(np.float32)
    k = rng.standard_normal((W * Tq, H * HD)).astype(np.float32)
    s = oracle.bmmQK(T(q, W * Tq, H * HD), T(k, W * Tq, H * HD), None, H, HD, W).array()
    q4 = q.reshape(W, Tq, H, HD).astype(np.float64)
    k4 = k.reshape(W, Tq, H, HD).astype(np.float64)
    ref = np.einsum("wihd,wjhd->whij", q4, k4).reshape(W * H * Tq, Tq)
    assert np.abs(s - ref).max() < 1e-5
    pv = oracle.bmmPV(T(s, W * H * Tq, Tq), T(k, W * Tq, H * HD), H, HD, W).array()
    refpv = np.einsum("whij,wjhd->wihd", ref.reshape(W, H, Tq, Tq), k4).reshape(W * Tq, H * HD)
    assert np.abs(pv - refpv).max() < 1e-4
