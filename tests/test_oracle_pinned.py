"""Pins the CPU oracle to outputs of the reference itself.

tests/golden/wasm_ref_outputs.npz holds what the reference's own compiled kernels returned
(src/gpu/wasm-kernels.wasm and src/engines/asr-parakeet/parakeet-decoder.wasm, executed by
oracle/wasm_exec.py; generator: tests/golden/gen_wasm_golden.py).  The C restatement under oracle/ must
reproduce every array bit for bit.  Where a reference checkout is present the small cases are also
re-executed live, so the fixture itself is checked against the module.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import pytest

from oracle.ref_wasm import reference_root
from oracle.wasm_oracle import LIB, _b, _f
from tests.golden.gen_wasm_golden import OUT, decoder_cases, kernel_cases, run_kernel_case


class PortKernels:
    """The four kernels of oracle/wasm_kernels_port.c with the argument meaning of RefWasmKernels."""

    def matmul_f32(self, a, b):
        M, K = a.shape
        N = b.shape[1]
        c = np.empty((M, N), np.float32)
        LIB.wk_matmul_f32(_f(np.ascontiguousarray(a)), _f(np.ascontiguousarray(b)), _f(c), M, K, N)
        return c

    def matmul_int8(self, a, wq, scale, N, K):
        M = a.shape[0]
        y = np.empty((M, N), np.float32)
        LIB.wk_matmul_int8(_f(np.ascontiguousarray(a)), _b(wq.view(np.uint8)), _f(scale), _f(y), M, N, K)
        return y

    def matmul_nbits(self, a, bq, scales, zp, N, block_size=32):
        M, K = a.shape
        nblk = -(-K // block_size)
        y = np.empty((M, N), np.float32)
        LIB.wk_matmul_nbits(_f(np.ascontiguousarray(a)), _b(bq), _f(scales), _b(zp), _f(y), M, N, K, nblk,
                            -(-nblk // 2), block_size)
        return y

    def conv1d_f32(self, x, w, cout, k, stride=1, pad_left=0, pad_right=0, dilation=1, groups=1):
        Cin, L = x.shape
        Lout = (L + pad_left + pad_right - dilation * (k - 1) - 1) // stride + 1
        y = np.empty((cout, Lout), np.float32)
        LIB.wk_conv1d_f32(_f(np.ascontiguousarray(x)), _f(np.ascontiguousarray(w).reshape(-1)), _f(y), cout, Cin, L,
                          Lout, k, stride, pad_left, dilation, groups)
        return y


@pytest.fixture(scope="module")
def golden():
    assert os.path.exists(OUT), "run python -m tests.golden.gen_wasm_golden on a machine with the reference"
    return np.load(OUT)


CASES = list(kernel_cases())


@pytest.mark.parametrize("name,kind,args", CASES, ids=[c[0] for c in CASES])
def test_port_matches_reference_wasm_bit_for_bit(golden, name, kind, args):
    got = run_kernel_case(PortKernels(), kind, args)
    ref = golden[name]
    assert got.shape == ref.shape
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), f"{name}: max diff {np.abs(got - ref).max()}"


def test_tdt_port_matches_reference_decoder_wasm(golden):
    from oracle.tdt_oracle import TdtOracle, synth_tdt_weights

    w = synth_tdt_weights(5)
    emitted = 0
    for name, int8, entry, frames, tenc in decoder_cases():
        o = TdtOracle(w, int8=int8)
        ids, fr = getattr(o, entry)(frames, tenc)
        assert np.array_equal(ids, golden[name + ".ids"]), name
        assert np.array_equal(fr, golden[name + ".frames"]), name
        emitted += len(ids)
        # the generator found the restatement's final 8198 logits, byte for byte, in the module's memory
        assert bool(golden[name + ".logits_found"][0]), name
        assert np.array_equal(o.last_logits().view(np.uint32), golden[name + ".logits"].view(np.uint32)), name
    assert emitted >= 3, "the cases must emit tokens to exercise predict / commit / the predproj cache"


LIVE = [c for c in CASES if c[0] in ("gate.matmul_none", "gate.matmulV3", "gate.matmulInt8", "gate.matmulNBits",
                                      "extra.matmul_3x5x7", "extra.int8_33x70x40", "extra.nbits_K100",
                                      "extra.conv1d_depthwise_k9", "extra.conv1d_grouped_s2_d2")]


@pytest.mark.skipif(reference_root() is None, reason="no reference checkout on this machine")
@pytest.mark.parametrize("name,kind,args", LIVE, ids=[c[0] for c in LIVE])
def test_fixture_is_what_the_shipped_module_returns(golden, name, kind, args):
    from oracle.ref_wasm import RefWasmKernels

    live = run_kernel_case(RefWasmKernels(), kind, args)
    assert np.array_equal(live.view(np.uint32), golden[name].view(np.uint32))
    assert np.array_equal(live.view(np.uint32), run_kernel_case(PortKernels(), kind, args).view(np.uint32))
