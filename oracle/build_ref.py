"""Compile the reference's own csrc/i8gemm.cpp (dense W8A8 linear) into oracle/_ref/ for validation.

Usage: REFERENCE_ROOT=/path/to/fused_cpp python oracle/build_ref.py
Only possible where the reference checkout exists; the built module travels with the repository
snapshot (oracle/_ref/ is ignored by git, not by the GPU runner) and is loaded by file name.
The MoE kernels of the reference are AArch64-only and are not buildable on an x86 host.
"""
from __future__ import annotations

import glob
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
NAME = "fused_cpp_ref_i8gemm"


def built_module_path() -> str | None:
    matches = sorted(glob.glob(os.path.join(OUT_DIR, NAME + "*.so")))
    return matches[0] if matches else None


def load_built():
    """Import the prebuilt module, or return None when it was never built."""
    path = built_module_path()
    if path is None:
        return None
    import torch  # noqa: F401  (the extension links libtorch)

    spec = importlib.util.spec_from_file_location(NAME, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def build(force: bool = False) -> str | None:
    root = os.environ.get("REFERENCE_ROOT", "/root/reference")
    source = os.path.join(root, "csrc", "i8gemm.cpp")
    if not os.path.exists(source):
        return built_module_path()
    if not force and built_module_path() is not None:
        return built_module_path()
    from torch.utils import cpp_extension

    # A toolchain wrapper exported as CXX may lack libgomp's spec file; the system compiler has it.
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    os.makedirs(OUT_DIR, exist_ok=True)
    cpp_extension.load(name=NAME, sources=[source, os.path.join(HERE, "i8gemm_ref_bind.cpp")], build_directory=OUT_DIR,
                       extra_cflags=["-O2", "-fopenmp", "-march=x86-64-v3"], extra_ldflags=["-fopenmp"], verbose=False)
    return built_module_path()


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
