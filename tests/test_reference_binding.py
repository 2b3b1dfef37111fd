"""The torch-extension binding shown in INTEGRATION.md (fused_cpp_b200/csrc/reference_binding/w8a8_b200.cpp) is valid
C++ against the torch headers and the C ABI header: a syntax-only compile, no GPU and no linking."""
from __future__ import annotations

import os
import shutil
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_side_binding_compiles_against_torch_headers():
    compiler = shutil.which("g++")
    cuda_include = "/usr/local/cuda/include"
    if compiler is None or not os.path.isdir(cuda_include):
        pytest.skip("needs g++ and the CUDA headers")
    torch_include = os.path.join(os.path.dirname(torch.__file__), "include")
    source = os.path.join(ROOT, "fused_cpp_b200", "csrc", "reference_binding", "w8a8_b200.cpp")
    command = [compiler, "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), "-I", torch_include,
               "-I", os.path.join(torch_include, "torch", "csrc", "api", "include"), "-I", cuda_include, source]
    result = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-4000:]
