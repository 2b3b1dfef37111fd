"""The DeepSeek-V4 attention-projection wrappers (fused_cpp_b200.deepseek_v4_w8a8) on the GPU: the weight quantiser
against the reference's formula (src/fused_cpp/deepseek_v4_w8a8.py:43-53), the linear and the paired linear against
the oracle's dense W8A8 GEMM (bit-exact), and the reference's argument checks."""
from __future__ import annotations

import pytest
import torch

from fused_cpp_b200 import deepseek_v4_w8a8 as w8a8
from oracle import oracle

pytestmark = pytest.mark.gpu


def _weight_reference(weight: torch.Tensor):
    fp32 = weight.float()
    maximum = fp32.abs().amax(dim=1, keepdim=True)
    scale = torch.where(maximum > 0, maximum / 127.0, torch.ones_like(maximum))
    return (fp32 / scale).round().clamp(-127, 127).to(torch.int8), scale.squeeze(1)


@pytest.mark.parametrize("n,k", [(48, 64), (7, 19), (130, 7168), (5, 16)])
def test_weight_quantiser_matches_reference_formula(cuda_device, n, k):
    generator = torch.Generator().manual_seed(n * 1000 + k)
    weight = (torch.randn((n, k), generator=generator) * 0.05).to(torch.bfloat16)
    weight[n // 2] = 0  # an all-zero channel takes scale 1
    prepared = w8a8.prepare_deepseek_v4_w8a8_linear_weight(weight)
    expected_q, expected_scale = _weight_reference(weight)
    assert (prepared.k, prepared.n) == (k, n)
    assert torch.equal(prepared.packed.packed_weight[:, :k].cpu(), expected_q)
    assert torch.equal(prepared.packed.weight_scale.cpu(), expected_scale)


def test_linear_and_pair_match_oracle(cuda_device):
    generator = torch.Generator().manual_seed(77)
    k = 200
    x = torch.randn((37, k), generator=generator).to(torch.bfloat16)
    first_w = (torch.randn((96, k), generator=generator) * 0.1).to(torch.bfloat16)
    second_w = (torch.randn((33, k), generator=generator) * 0.1).to(torch.bfloat16)
    first = w8a8.prepare_deepseek_v4_w8a8_linear_weight(first_w)
    second = w8a8.prepare_deepseek_v4_w8a8_linear_weight(second_w.to(cuda_device))  # CUDA source weights are accepted
    q1, s1 = _weight_reference(first_w)
    q2, s2 = _weight_reference(second_w)
    out = w8a8.deepseek_v4_w8a8_linear(x.to(cuda_device), first)
    torch.testing.assert_close(out.cpu(), oracle.i8gemm_dynamic(x, q1, s1, None, torch.bfloat16), atol=0, rtol=0)
    buffer = torch.empty_like(out)
    assert w8a8.deepseek_v4_wo_b_w8a8(x.to(cuda_device), first, out=buffer) is buffer
    assert torch.equal(buffer, out)
    batched = w8a8.deepseek_v4_w8a8_linear(x.reshape(1, 37, k).to(cuda_device), first)
    assert batched.shape == (1, 37, 96) and torch.equal(batched[0], out)
    a, b = w8a8.deepseek_v4_w8a8_linear_pair(x.to(cuda_device), first, second)
    torch.testing.assert_close(a.cpu(), oracle.i8gemm_dynamic(x, q1, s1, None, torch.bfloat16, clamp_low=-127), atol=0, rtol=0)
    torch.testing.assert_close(b.cpu(), oracle.i8gemm_dynamic(x, q2, s2, None, torch.bfloat16, clamp_low=-127), atol=0, rtol=0)


def test_checkpoint_int8_weights_and_argument_checks(cuda_device):
    generator = torch.Generator().manual_seed(3)
    q = torch.randint(-127, 128, (24, 64), dtype=torch.int8, generator=generator)
    scale = torch.rand(24, generator=generator) * 0.01 + 0.001
    prepared = w8a8.prepare_deepseek_v4_w8a8_linear_quantized_weight(q, scale, backend="sve")
    x = torch.randn((5, 64), generator=generator).to(torch.bfloat16)
    out = w8a8.deepseek_v4_w8a8_linear(x.to(cuda_device), prepared)
    torch.testing.assert_close(out.cpu(), oracle.i8gemm_dynamic(x, q, scale, None, torch.bfloat16), atol=0, rtol=0)
    with pytest.raises(TypeError, match="must be PreparedDeepSeekV4W8A8LinearWeight"):
        w8a8.deepseek_v4_w8a8_linear(x.to(cuda_device), prepared.packed)
    with pytest.raises(TypeError, match="CUDA torch.bfloat16"):
        w8a8.deepseek_v4_w8a8_linear(x, prepared)
    with pytest.raises(ValueError, match="input K must be 64"):
        w8a8.deepseek_v4_w8a8_linear(torch.zeros((2, 32), dtype=torch.bfloat16, device=cuda_device), prepared)
    with pytest.raises(ValueError, match="non-negative"):
        w8a8.deepseek_v4_w8a8_linear(x.to(cuda_device), prepared, num_threads=-1)
    with pytest.raises(TypeError, match="torch.int8"):
        w8a8.prepare_deepseek_v4_w8a8_linear_quantized_weight(q.float(), scale)
    with pytest.raises(ValueError, match="must contain N=24"):
        w8a8.prepare_deepseek_v4_w8a8_linear_quantized_weight(q, scale[:3])
    with pytest.raises(TypeError, match="torch.bfloat16"):
        w8a8.prepare_deepseek_v4_w8a8_linear_weight(q.float())
    with pytest.raises(ValueError, match="share K"):
        other = w8a8.prepare_deepseek_v4_w8a8_linear_quantized_weight(q[:, :32].contiguous(), scale)
        w8a8.deepseek_v4_w8a8_linear_pair(x.to(cuda_device), prepared, other)
