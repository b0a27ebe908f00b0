"""Build recipe for the CPU oracle (test infrastructure; never part of the product).

    python oracle/build_oracle.py

Compiles oracle/wasm_kernels_port.c, oracle/parakeet_decoder_port.c and oracle/nemo_mel_port.c into oracle/liboracle.so.  -ffp-contract=off keeps
every multiply and add separately rounded, as wasm32 simd128 does; -O3 changes no
floating-point result without -ffast-math.  OpenMP (used only by the *_mt / *_kj
entry points and conv2d, all bit-identical to their serial forms) is enabled when the
compiler has a working libgomp, else those entry points run on one thread.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRCS = [os.path.join(HERE, "wasm_kernels_port.c"), os.path.join(HERE, "parakeet_decoder_port.c"),
        os.path.join(HERE, "nemo_mel_port.c")]
OUT = os.path.join(HERE, "liboracle.so")
BASE = ["-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-fvisibility=hidden",
        "-Wall", "-Wextra", "-shared"]


def _compilers():
    seen = []
    for cc in ("/usr/bin/gcc", os.environ.get("CC"), shutil.which("gcc"), shutil.which("cc")):
        if cc and cc not in seen and os.path.exists(cc):
            seen.append(cc)
    return seen


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= max(os.path.getmtime(s) for s in SRCS):
        return OUT
    errors = []
    for omp in (["-fopenmp"], []):
        for cc in _compilers():
            cmd = [cc, *BASE, *omp, "-o", OUT, *SRCS, "-lm"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                return OUT
            errors.append(" ".join(cmd) + "\n" + r.stderr[-400:])
    raise RuntimeError("oracle build failed:\n" + "\n".join(errors))


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
