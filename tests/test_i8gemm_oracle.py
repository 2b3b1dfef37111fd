"""Dense W8A8 linear: the oracle's restatement against (1) golden outputs of the reference's own test
reference and (2) the reference's own csrc/i8gemm.cpp compiled into oracle/_ref (when that was built)."""
from __future__ import annotations

import os

import pytest
import torch

from oracle import build_ref, oracle
from tests import cases

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", sorted(cases.I8GEMM_CASES))
def test_oracle_matches_reference_test_function(name):
    case = cases.i8gemm_case(name)
    golden = torch.load(os.path.join(GOLDEN, f"i8gemm_{name}.pt"))["out"]
    out = oracle.i8gemm_dynamic(case["x"], case["weight"], case["weight_scale"], case["bias"], case["out_dtype"])
    assert out.dtype == golden.dtype
    torch.testing.assert_close(out, golden, atol=0, rtol=0)  # the reference's own test uses atol=0 (tests/test_i8gemm.py:61)


@pytest.mark.parametrize("name", sorted(cases.I8GEMM_CASES))
def test_oracle_matches_compiled_reference(name):
    reference = build_ref.load_built()
    if reference is None:
        pytest.skip("oracle/_ref was not built in this checkout (needs the reference sources)")
    case = cases.i8gemm_case(name)
    packed, scale, k, n, kp, np_, backend = reference.i8gemm_prepare(case["weight"], case["weight_scale"], "auto")
    assert backend == "fallback"
    out_ref = torch.empty((case["x"].shape[0], n), dtype=case["out_dtype"])
    reference.i8gemm_dynamic_scaled_mm(out_ref, case["x"].contiguous(), packed, scale, case["bias"], k, n, kp, np_, 0)
    out = oracle.i8gemm_dynamic(case["x"], case["weight"], case["weight_scale"], case["bias"], case["out_dtype"])
    torch.testing.assert_close(out, out_ref, atol=0, rtol=0)
    if case["x"].dtype == torch.bfloat16:
        first = torch.empty((case["x"].shape[0], n), dtype=torch.bfloat16)
        second = torch.empty_like(first)
        reference.i8gemm_dynamic_scaled_mm_pair(first, second, case["x"].contiguous(), packed, scale, k, n, kp, np_, packed, scale, n, np_, 0)
        pair = oracle.i8gemm_dynamic(case["x"], case["weight"], case["weight_scale"], None, torch.bfloat16, clamp_low=-127)
        torch.testing.assert_close(pair, first, atol=0, rtol=0)
        torch.testing.assert_close(pair, second, atol=0, rtol=0)
