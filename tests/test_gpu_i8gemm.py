"""Dense W8A8 linear on the GPU through fused_cpp_b200.i8gemm, against the oracle and the reference golden
(exact: int32 accumulation on the tensor cores, the same fp32 dequant order)."""
from __future__ import annotations

import os

import pytest
import torch

from fused_cpp_b200 import i8gemm
from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", sorted(cases.I8GEMM_CASES))
def test_dynamic_scaled_mm_matches_reference(cuda_device, name):
    case = cases.i8gemm_case(name)
    packed = i8gemm.prepare(case["weight"], case["weight_scale"])
    assert packed.backend == "cuda_sm100_tcgen05" and packed.k_padded % 16 == 0
    bias = None if case["bias"] is None else case["bias"].to(cuda_device)
    out = i8gemm.dynamic_scaled_mm(case["x"].to(cuda_device), packed, bias=bias, out_dtype=case["out_dtype"])
    expected = oracle.i8gemm_dynamic(case["x"], case["weight"], case["weight_scale"], case["bias"], case["out_dtype"])
    golden = torch.load(os.path.join(GOLDEN, f"i8gemm_{name}.pt"))["out"]
    assert out.dtype == case["out_dtype"] and tuple(out.shape) == tuple(golden.shape)
    torch.testing.assert_close(out.cpu(), expected, atol=0, rtol=0)
    torch.testing.assert_close(out.cpu(), golden, atol=0, rtol=0)


def test_batched_input_scalar_scale_and_empty(cuda_device):
    """tests/test_i8gemm.py:64-80 of the reference: leading batch dims and a scalar weight scale."""
    generator = torch.Generator().manual_seed(1)
    weight = torch.randint(-8, 9, (11, 19), dtype=torch.int8, generator=generator)
    scale = torch.tensor(0.02)
    x = torch.randn((2, 3, 19), generator=generator)
    packed = i8gemm.prepare(weight, scale)
    out = i8gemm.dynamic_scaled_mm(x.to(cuda_device), packed, out_dtype=torch.float32)
    expected = oracle.i8gemm_dynamic(x.reshape(-1, 19), weight, scale, None, torch.float32).reshape(2, 3, 11)
    torch.testing.assert_close(out.cpu(), expected, atol=0, rtol=0)
    assert i8gemm.dynamic_scaled_mm(x[:0].to(cuda_device), packed).shape == (0, 3, 11)
    with pytest.raises(RuntimeError, match="x last dim must be K=19"):
        i8gemm.dynamic_scaled_mm(torch.zeros((2, 20), device=cuda_device), packed)


def test_pair_shares_one_quantisation(cuda_device):
    case = cases.i8gemm_case("wide")
    other = cases.i8gemm_case("deep")
    first = i8gemm.prepare(case["weight"], case["weight_scale"])
    second_weight = other["weight"][:, :300].contiguous()
    second = i8gemm.prepare(second_weight, other["weight_scale"])
    a, b = i8gemm.dynamic_scaled_mm_pair(case["x"].to(cuda_device), first, second)
    ea = oracle.i8gemm_dynamic(case["x"], case["weight"], case["weight_scale"], None, torch.bfloat16, clamp_low=-127)
    eb = oracle.i8gemm_dynamic(case["x"], second_weight, other["weight_scale"], None, torch.bfloat16, clamp_low=-127)
    torch.testing.assert_close(a.cpu(), ea, atol=0, rtol=0)
    torch.testing.assert_close(b.cpu(), eb, atol=0, rtol=0)
