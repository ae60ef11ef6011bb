"""Compile the CPU oracle (``oracle/trigrad_oracle.cpp``) into ``oracle/libtrigrad_oracle.so``.

TEST INFRASTRUCTURE ONLY.  ``-ffp-contract=off`` is essential: the oracle fixes FMA placement
explicitly with ``fmaf`` and must not let the compiler add more; ``-mfma`` only makes those
explicit calls one instruction instead of a libm call.

Usage: python oracle/build.py [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "trigrad_oracle.cpp")
LIB = os.path.join(HERE, "libtrigrad_oracle.so")


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-mfma", "-fopenmp", "-shared", "-fPIC",
           "-Wall", "-Wno-unknown-pragmas", SRC, "-o", LIB]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
