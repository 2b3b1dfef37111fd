"""Build the CPU oracle (test infrastructure) into oracle/_build/libmoe_oracle.so.

Usage: python oracle/build.py
The flags are part of the oracle's definition: contraction must stay off so that only the
multiply-adds written as fmaf() are fused, exactly where the reference fuses them.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libmoe_oracle.so")
SRC = os.path.join(HERE, "moe_oracle.c")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = [
        "gcc", "-O2", "-march=x86-64-v3", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
        "-std=c11", "-shared", "-fPIC", "-o", LIB, SRC, "-lm",
    ]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
