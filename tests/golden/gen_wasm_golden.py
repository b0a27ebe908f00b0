"""Generates tests/golden/wasm_ref_outputs.npz: outputs of the REFERENCE's own compiled kernels.

    python -m tests.golden.gen_wasm_golden          (needs a reference checkout; a few minutes)

The shipped modules ``src/gpu/wasm-kernels.wasm`` and ``src/engines/asr-parakeet/parakeet-decoder.wasm``
are executed by oracle/wasm_exec.py through the reference's host calling convention (oracle/ref_wasm.py)
on the inputs ``kernel_cases()`` / ``decoder_cases()`` below define, and what they return is stored.
tests/test_oracle_pinned.py then requires the C restatement under oracle/ to reproduce every array bit
for bit, which pins the oracle to outputs of the reference itself.  Inputs are not stored: both sides
rebuild them from the seeds here (mulberry32(0x5eed) in the draw order of
scripts/backend-conformance.mjs:46-141 for the gate's own cases, numpy PCG64 for the added ones).
"""
from __future__ import annotations

import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "wasm_ref_outputs.npz")


def kernel_cases():
    """Yields (name, kind, args) for the four exports of wasm-kernels.wasm."""
    from oracle.wasm_oracle import Mulberry32

    g = Mulberry32(0x5EED)

    def data(r, c):
        return g.data(r * c).reshape(r, c)

    # the matmul-family cases of the reference gate, in its draw order (bias/add drawn but unused here:
    # the module computes bare accumulations, the JS host applies bias/activation/residual afterwards)
    for act in ["none", "gelu", "gelu_erf", "tanh", "relu", "silu"]:
        a, b, _ = data(37, 53), data(53, 41), data(1, 41)
        yield f"gate.matmul_{act}", "matmul_f32", (a, b)
    a, b, _ = data(64, 128), data(128, 256), data(64, 256)
    yield "gate.matmul_relu_add", "matmul_f32", (a, b)
    a, b = data(33, 48), data(48, 52)
    yield "gate.matmulV2", "matmul_f32", (a, b)
    a, b = data(33, 64), data(64, 48)
    yield "gate.matmulV3", "matmul_f32", (a, b)
    a, b, _ = data(129, 64), data(64, 132), data(1, 132)
    yield "gate.matmulV4", "matmul_f32", (a, b)
    a, b = data(40, 64), data(64, 64)
    yield "gate.matmulF16", "matmul_f32", (a, b)
    a, b, _ = data(65, 128), data(128, 256), data(1, 256)
    yield "gate.matmul_f16B", "matmul_f32", (a, b)
    a = data(9, 20)
    packed = g.bytes(20 * 16)
    s, _ = data(1, 16), data(1, 16)
    yield "gate.matmulInt8", "matmul_int8", (a, packed, s.reshape(-1), 16, 20)
    a = data(7, 64)
    bq = g.bytes(8 * 2 * 16)
    zp = g.bytes(8 * 1 * 4)
    s = data(1, 16)
    yield "gate.matmulNBits", "matmul_nbits", (a, bq, s.reshape(-1), zp, 8)

    # added cases: ragged shapes, the partial last block of scripts/wasm-verify.mjs:199-228 (K = 100),
    # int8 weights over the full [-128,127] byte range, depthwise / grouped / strided / dilated conv1d
    rng = np.random.default_rng(1234)
    a = rng.standard_normal((3, 5)).astype(np.float32)
    b = rng.standard_normal((5, 7)).astype(np.float32)
    yield "extra.matmul_3x5x7", "matmul_f32", (a, b)
    a = rng.standard_normal((17, 96)).astype(np.float32)
    b = (rng.standard_normal((96, 70)) * 100).astype(np.float32)
    yield "extra.matmul_17x96x70", "matmul_f32", (a, b)
    a = rng.standard_normal((33, 70)).astype(np.float32)
    wq = rng.integers(0, 256, 70 * 40, dtype=np.uint8)
    s = rng.uniform(1e-3, 1e-2, 40).astype(np.float32)
    yield "extra.int8_33x70x40", "matmul_int8", (a, wq, s, 40, 70)
    M, K, N = 5, 100, 12
    nblk = 4
    a = rng.standard_normal((M, K)).astype(np.float32)
    bq = rng.integers(0, 256, N * nblk * 16, dtype=np.uint8)
    zp = rng.integers(0, 256, N * 2, dtype=np.uint8)
    s = rng.uniform(5e-3, 2e-2, N * nblk).astype(np.float32)
    yield "extra.nbits_K100", "matmul_nbits", (a, bq, s, zp, N)
    M, K, N = 4, 256, 24
    nblk = 8
    a = rng.standard_normal((M, K)).astype(np.float16).astype(np.float32)
    bq = rng.integers(0, 256, N * nblk * 16, dtype=np.uint8)
    zp = np.full(N * 4, 0x88, np.uint8)
    s = rng.uniform(5e-3, 2e-2, N * nblk).astype(np.float16).astype(np.float32)
    yield "extra.nbits_decode_like", "matmul_nbits", (a, bq, s, zp, N)
    x = rng.standard_normal((16, 50)).astype(np.float32)
    w = rng.standard_normal((16, 9)).astype(np.float32)
    w[3, 4] = 0.0  # the kernel skips taps whose weight is exactly zero
    yield "extra.conv1d_depthwise_k9", "conv1d_f32", (x, w, dict(cout=16, k=9, pad_left=4, pad_right=4, groups=16))
    x = rng.standard_normal((8, 41)).astype(np.float32)
    w = rng.standard_normal((12, 2 * 3)).astype(np.float32)
    yield "extra.conv1d_grouped_s2_d2", "conv1d_f32", (x, w, dict(cout=12, k=3, stride=2, pad_left=1, pad_right=2, dilation=2, groups=4))


def decoder_cases():
    """Yields (name, int8, entry, frames, tenc); weights come from oracle.tdt_oracle.synth_tdt_weights(5)."""
    rng = np.random.default_rng(77)
    proj = rng.standard_normal((6, 640)).astype(np.float32)
    yield "tdt.decode_proj_int8", True, "decode_proj", proj, 6
    frames = rng.standard_normal((3, 1024)).astype(np.float32)
    frames[1, ::7] = 0.0  # the projection skips frame entries that are exactly zero
    yield "tdt.decode_f32", False, "decode", frames, 3


def run_kernel_case(backend, kind, args):
    """backend: RefWasmKernels (the reference) or PortKernels (the C restatement)."""
    if kind == "matmul_f32":
        return backend.matmul_f32(*args)
    if kind == "matmul_int8":
        return backend.matmul_int8(*args)
    if kind == "matmul_nbits":
        return backend.matmul_nbits(*args)
    x, w, kw = args
    return backend.conv1d_f32(x, w, **kw)


def find_f32_block(mem: bytes, block: np.ndarray) -> int:
    """Offset at which linear memory holds exactly these f32 values, or -1."""
    return bytes(mem).find(np.ascontiguousarray(block, np.float32).tobytes())


def main():
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle.ref_wasm import RefWasmKernels, RefWasmTdtDecoder
    from oracle.tdt_oracle import TdtOracle, synth_tdt_weights

    out = {}
    ref = RefWasmKernels()
    for name, kind, args in kernel_cases():
        t = time.time()
        out[name] = run_kernel_case(ref, kind, args)
        print(f"{name}: {out[name].shape} in {time.time() - t:.1f}s", flush=True)
    w = synth_tdt_weights(5)
    for name, int8, entry, frames, tenc in decoder_cases():
        t = time.time()
        dec = RefWasmTdtDecoder(w, int8=int8)
        ids, fr = getattr(dec, entry)(frames, tenc)
        out[name + ".ids"], out[name + ".frames"] = ids, fr
        # the module does not export its logits; they sit in its static data, so look the restatement's
        # final logits up in the module's linear memory: found = bit-identical, all 8198 of them
        o = TdtOracle(w, int8=int8)
        getattr(o, entry)(frames, tenc)
        out[name + ".logits_found"] = np.array([find_f32_block(dec.inst.mem, o.last_logits()) >= 0])
        out[name + ".logits"] = o.last_logits() if out[name + ".logits_found"][0] else np.zeros(0, np.float32)
        print(f"{name}: ids {ids.tolist()} frames {fr.tolist()} logits in module memory: "
              f"{bool(out[name + '.logits_found'][0])} in {time.time() - t:.1f}s", flush=True)
    np.savez_compressed(OUT, **out)
    print(OUT, len(out), "arrays", os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
