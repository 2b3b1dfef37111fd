"""Build libfused_moe_b200.so (and its diagnostic twin) in-tree with nvcc for sm_100a.

Usage: python -m fused_cpp_b200.build [--force] [--verbose]
The library links only the CUDA runtime (statically); it has no torch dependency, so it builds
in seconds and the same file serves Python (ctypes) and any other C-ABI caller.

Two files come out:
  lib/libfused_moe_b200.so       the product: the tcgen05 kernels and the C ABI of include/fused_moe_b200.h;
  lib/libfused_moe_b200_diag.so  the same sources compiled with -DFMOE_DIAG plus a CUDA-core cross-check GEMM and
                                 a tensor-core issue-rate probe (csrc/diag.h).  Only tests and measurement
                                 scripts load it; nothing in the package's forward path does.
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
DIAG_LIB = os.path.join(OUT_DIR, "libfused_moe_b200_diag.so")
SOURCES = ["api.cu", "route.cu", "quant.cu", "merge.cu", "umma_gemm.cu", "umma2_gemm.cu", "ep.cu", "router.cu"]
DIAG_ONLY_SOURCES = ["simt_gemm.cu", "probe.cu"]
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
    newest = _newest_input()
    if not force and all(os.path.exists(p) and os.path.getmtime(p) >= newest for p in (LIB, DIAG_LIB)):
        return LIB
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(job) -> str:
        name, diag = job
        obj = os.path.join(OUT_DIR, ("diag_" if diag else "") + name.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *(["-DFMOE_DIAG"] if diag else []), *extra, "-c", os.path.join(CSRC, name), "-o", obj]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}")
        return obj

    jobs = [(name, False) for name in SOURCES] + [(name, True) for name in SOURCES + DIAG_ONLY_SOURCES]
    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
        objects = list(pool.map(compile_one, jobs))
    product = objects[: len(SOURCES)]
    diagnostic = objects[len(SOURCES):]
    for target, parts in ((LIB, product), (DIAG_LIB, diagnostic)):
        subprocess.run([nvcc, "-shared", "-o", target, *parts, "-gencode", "arch=compute_100a,code=sm_100a"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
