"""CPU-side checks of the boundary: the library loads without a GPU, exports every symbol the
header declares, and refuses to create a context when no device exists (no CPU fallback)."""
import ctypes
import os

import pytest


def test_library_exports_every_declared_symbol(pkg):
    from fluidaudio_web_b200 import _lib

    lib = pkg.load_library()
    declared = _lib.declared_symbols()
    assert len(declared) >= 50
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/fa_cuda.h but not exported"
    # every bound signature is declared too (binding and header stay in sync)
    assert set(_lib.SIGNATURES) | {"fa_last_error"} == set(declared)


def test_no_cpu_fallback(pkg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.CudaError) as ei:
        pkg.CudaContext(0)
    assert "no CUDA device" in str(ei.value) and "no CPU fallback" in str(ei.value)


def test_product_package_does_not_import_oracle():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkgdir = os.path.join(root, "fluidaudio-web_b200")
    for dirpath, _dirs, files in os.walk(pkgdir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


def test_missing_library_fails_loudly(pkg, monkeypatch):
    from fluidaudio_web_b200 import _lib

    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "library_path", lambda: "/nonexistent/libfa_cuda.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load_library()
