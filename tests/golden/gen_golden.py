"""Generates tests/golden/conformance_gemm.npz.

    python -m tests.golden.gen_golden

The reference ships no golden vectors for its GEMMs and cannot run in the build
container, so these fixtures are the CPU oracle's outputs on the reference gate's own
seeded inputs: the matmul-family cases of scripts/backend-conformance.mjs:67-141, drawn
from mulberry32(0x5eed) in the script's order (one shared generator across cases).
They freeze the oracle (a regression pin) and give the GPU tests fixed inputs/outputs
that do not depend on a compiler being present.
"""
from __future__ import annotations

import os

import numpy as np


def conformance_gemm_cases(oracle):
    """Yields (name, inputs dict, oracle output [M,N] f32) in the gate's draw order."""
    from oracle.wasm_oracle import Mulberry32, T

    g = Mulberry32(0x5EED)

    def pair(r, c):
        return T(g.data(r * c), r, c)

    # :67-74  six activations, odd shape 37x53x41 with bias
    for act in ["none", "gelu", "gelu_erf", "tanh", "relu", "silu"]:
        a, b, bias = pair(37, 53), pair(53, 41), pair(1, 41)
        yield (f"matmul_bias_{act}", dict(a=a.array(), b=b.array(), bias=bias.array(), act=act),
               oracle.matmul(a, b, bias=bias, act=act).array())
    # :75-80  vec4 shape + fused add
    a, b, d = pair(64, 128), pair(128, 256), pair(64, 256)
    yield "matmul_relu_add", dict(a=a.array(), b=b.array(), add=d.array(), act="relu"), oracle.matmul(a, b, act="relu", add=d).array()
    # :81-85 V2
    a, b = pair(33, 48), pair(48, 52)
    yield "matmulV2_gelu", dict(a=a.array(), b=b.array(), act="gelu"), oracle.matmulV2(a, b, act="gelu").array()
    # :86-90 V3
    a, b = pair(33, 64), pair(64, 48)
    yield "matmulV3", dict(a=a.array(), b=b.array(), act="none"), oracle.matmulV3(a, b).array()
    # :91-96 V4
    a, b, bias = pair(129, 64), pair(64, 132), pair(1, 132)
    yield "matmulV4_bias_silu", dict(a=a.array(), b=b.array(), bias=bias.array(), act="silu"), oracle.matmulV4(a, b, bias=bias, act="silu").array()
    # :98-105 matmulF16 (f16 a/b/c on the GPU side; CPU twin is f32)
    ad, bd = g.data(40 * 64), g.data(64 * 64)
    yield "matmulF16", dict(a=ad.reshape(40, 64), b=bd.reshape(64, 64), act="none"), oracle.matmulF16(T(ad, 40, 64), T(bd, 64, 64)).array()
    # :106-114 f16-B route
    ad, bd = g.data(65 * 128), g.data(128 * 256)
    bias = pair(1, 256)
    yield "matmul_f16B_bias_silu", dict(a=ad.reshape(65, 128), b=bd.reshape(128, 256), bias=bias.array(), act="silu"), oracle.matmul(T(ad, 65, 128), T(bd, 128, 256), bias=bias, act="silu").array()
    # :119-128 matmulInt8 9x20x16, random bytes, bias+relu
    a = pair(9, 20)
    packed = g.bytes(20 * 16)
    s, bias = pair(1, 16), pair(1, 16)
    yield "matmulInt8_bias_relu", dict(a=a.array(), wq=packed, scale=s.array(), bias=bias.array(), act="relu", N=16, K=20), oracle.matmulInt8(a, oracle.uploadBytes(packed), s, 16, 20, bias=bias, act="relu").array()
    # :129-141 matmulNBits N=8 K=64 nblk=2
    N, K, nblk = 8, 64, 2
    a = pair(7, K)
    bq = g.bytes(N * nblk * 16)
    zp = g.bytes(N * ((nblk + 1) // 2) * 4)
    s = pair(1, N * nblk)
    yield "matmulNBits", dict(a=a.array(), bq=bq, zp=zp, scales=s.array(), N=N), oracle.matmulNBits(a, oracle.uploadBytes(bq), s, oracle.uploadBytes(zp), N).array()


def main():
    from oracle.wasm_oracle import WasmOracle

    out = {}
    for name, inputs, y in conformance_gemm_cases(WasmOracle()):
        out[name] = y
        for k, v in inputs.items():
            if isinstance(v, np.ndarray):
                out[f"{name}.in.{k}"] = v
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "conformance_gemm.npz")
    np.savez_compressed(path, **out)
    print(path, len(out), "arrays", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
