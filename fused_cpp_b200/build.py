"""Build libfused_moe_b200.so in-tree with nvcc for sm_100a.

Usage: python -m fused_cpp_b200.build [--force] [--verbose]
The library links only the CUDA runtime (statically); it has no torch dependency, so it builds
in seconds and the same file serves Python (ctypes) and any other C-ABI caller.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(OUT_DIR, "libfused_moe_b200.so")
SOURCES = ["api.cu", "route.cu", "quant.cu", "merge.cu", "simt_gemm.cu", "umma_gemm.cu", "umma2_gemm.cu", "ep.cu", "probe.cu", "router.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if candidate and (os.path.sep not in candidate or os.path.exists(candidate)):
            return candidate
    raise RuntimeError("nvcc not found")


def _newest_input() -> float:
    paths = [os.path.join(CSRC, name) for name in os.listdir(CSRC)]
    paths.append(os.path.join(os.path.dirname(HERE), "include", "fused_moe_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_input():
        return LIB
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(name: str) -> str:
        obj = os.path.join(OUT_DIR, name.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, name), "-o", obj]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objects = list(pool.map(compile_one, SOURCES))
    link = [nvcc, "-shared", "-o", LIB, *objects, "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
