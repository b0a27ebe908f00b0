import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.wasm_oracle import WasmOracle

    return WasmOracle()


@pytest.fixture(scope="session")
def pkg():
    """The product package (directory name has a hyphen, so it is loaded by path)."""
    import __graft_entry__ as ge

    return ge.load_package()


@pytest.fixture(scope="session")
def ctx(pkg):
    c = pkg.CudaContext(device=0)
    yield c
    c.destroy()
