"""BF16 routed-expert MoE on the GPU against the CPU oracle and the golden outputs of the reference's
fused_moe_naive.

Tolerances.  The tensor cores accumulate in fp32 in a different order than any CPU loop, so BF16 results
are compared to tolerance: relative L2 <= 5e-3 on the bf16 output, and max-abs <= 1e-2 x RMS on the
fp32 route rows (the values before the final bf16 rounding).  On the bf16 output itself one extra bf16
ulp of the element is allowed on top of 1e-2 x RMS, because two correctly rounded bf16 results of values
that differ by 1e-6 can land one ulp apart (an ulp of a 4-sigma element is already ~3e-2 x RMS).
"""
from __future__ import annotations

import os

import pytest
import torch

from fused_cpp_b200 import _lib
from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
IMPLS = {"simt": _lib.GEMM_SIMT, "umma": _lib.GEMM_UMMA}


def _run(case, device, **kw):
    c = {k: v.to(device) for k, v in case.items()}
    return _lib.moe_forward(c["x"], c["w13"], c["w2"], c["topk_weights"], c["topk_ids"], **kw)


def _assert_close_bf16(actual: torch.Tensor, expected: torch.Tensor, what: str):
    a, e = actual.float(), expected.float()
    rms = float(e.pow(2).mean().sqrt())
    rel_l2 = float((a - e).norm() / e.norm())
    assert rel_l2 <= 5e-3, f"{what}: relative L2 {rel_l2:.3e}"
    ulp = e.abs() * 2.0 ** -7
    excess = ((a - e).abs() - ulp).max()
    assert float(excess) <= 1e-2 * rms, f"{what}: max-abs beyond one bf16 ulp is {float(excess):.3e} vs RMS {rms:.3e}"


@pytest.mark.parametrize("impl", ["simt", "umma"])
@pytest.mark.parametrize("limit", [0.0, 10.0], ids=["silu", "clamp10"])
@pytest.mark.parametrize("name", cases.BF16_CASES)
def test_bf16_matches_oracle(cuda_device, name, limit, impl):
    case = cases.bf16_case(name)
    if limit:
        case["x"] = (case["x"].float() * 40).to(torch.bfloat16)  # push gate/up beyond the clamp
    result = _run(case, cuda_device, gemm_impl=IMPLS[impl], swiglu_limit=limit, dump=True)
    assert result.status()[0] == 0
    out_ref, d = oracle.bf16_forward(case["x"], case["w13"], case["w2"], case["topk_weights"], case["topk_ids"], limit, dumps=True)
    tokens, hidden = case["x"].shape
    top_k = case["topk_ids"].shape[1]
    routes = tokens * top_k
    experts = case["w13"].shape[0]
    counts, offsets, order = oracle.route_build(case["topk_ids"], experts)
    assert torch.equal(result.region("sorted_routes", torch.int32, (routes,)).cpu(), order)
    gathered = result.region("a_rows", torch.bfloat16, (routes, hidden)).cpu()
    assert torch.equal(gathered.view(torch.int16), case["x"][(order // top_k).long()].view(torch.int16))
    route_out = result.region("route_out", torch.float32, (routes, hidden)).cpu()
    rms = float(d["route_out"].pow(2).mean().sqrt())
    assert float((route_out - d["route_out"]).abs().max()) <= 1e-2 * rms
    assert float((route_out - d["route_out"]).norm() / d["route_out"].norm()) <= 5e-3
    # The merge itself is exact arithmetic on whatever route rows the GEMM produced.
    merged = oracle.merge_bf16_path(route_out.view(tokens, top_k, hidden), case["topk_weights"])
    assert torch.equal(result.out.cpu().view(torch.int16), merged.view(torch.int16)), "top-k merge order differs"
    _assert_close_bf16(result.out.cpu(), out_ref, "output vs oracle")


@pytest.mark.parametrize("name", cases.BF16_CASES)
def test_bf16_matches_reference_golden(cuda_device, name):
    """Golden = fused_cpp.moe.naive.fused_moe_naive of the reference in fp32, cast to bf16."""
    case = cases.bf16_case(name)
    golden = torch.load(os.path.join(GOLDEN, f"bf16_{name}.pt"))["out"]
    out = _run(case, cuda_device).out.cpu()
    rel_l2 = float((out.float() - golden.float()).norm() / golden.float().norm())
    assert rel_l2 <= 5e-3


def test_bf16_umma_matches_simt_route_rows(cuda_device):
    case = cases.bf16_case("top8")
    umma = _run(case, cuda_device, gemm_impl=_lib.GEMM_UMMA)
    rows_umma = umma.region("route_out", torch.float32, (case["topk_ids"].numel(), case["x"].shape[1])).clone()
    simt = _run(case, cuda_device, gemm_impl=_lib.GEMM_SIMT)
    rows_simt = simt.region("route_out", torch.float32, (case["topk_ids"].numel(), case["x"].shape[1]))
    assert float((rows_umma - rows_simt).norm() / rows_simt.norm()) <= 1e-3


@pytest.mark.parametrize("tile", [16, 64, 256, 512])
def test_bf16_repeat_and_tile_invariance(cuda_device, tile):
    """Same bits on a repeated call; per-row results do not depend on the row tile because each output
    element is one MMA column whose K order is fixed."""
    case = cases.bf16_case("wide")
    base = _run(case, cuda_device, gate_up_tile=128, down_tile=128).out.clone()
    again = _run(case, cuda_device, gate_up_tile=tile, down_tile=tile).out
    assert torch.equal(base.view(torch.int16), again.view(torch.int16))
