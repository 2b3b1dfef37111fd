"""The CPU oracle against the golden outputs of the reference's own Python functions (no GPU)."""
from __future__ import annotations

import math
import os

import pytest
import torch

from oracle import oracle
from tests import cases

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", cases.W8A8_CASES)
def test_w8a8_oracle_is_bit_exact_against_reference_python(name):
    case = cases.w8a8_case(name)
    golden = torch.load(os.path.join(GOLDEN, f"w8a8_{name}.pt"))
    out, d = oracle.w8a8_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"],
                                 case["topk_ids"], oracle.NUMERICS_TORCHREF, dumps=True)
    assert torch.equal(d["xq"], golden["xq"])
    assert torch.equal(d["a"], golden["a"].float())
    assert torch.equal(out.view(torch.int16), golden["out"].view(torch.int16))


@pytest.mark.parametrize("name", cases.W8A8_CASES)
def test_w8a8_native_numerics_stay_within_the_reference_tolerance(name):
    """The reference accepts atol=3e-6 between its native kernel and its Python reference on outputs of
    magnitude ~1e-4 (tests/test_moe_w8a8.py:225), i.e. a few bf16 ulps; hold the NATIVE restatement to
    two bf16 ulps of the output scale."""
    case = cases.w8a8_case(name)
    golden = torch.load(os.path.join(GOLDEN, f"w8a8_{name}.pt"))["out"].float()
    out = oracle.w8a8_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"],
                              case["topk_ids"], oracle.NUMERICS_NATIVE).float()
    scale = float(golden.abs().max())
    assert float((out - golden).abs().max()) <= 2.0 * scale * 2.0 ** -7


@pytest.mark.parametrize("name", cases.BF16_CASES)
def test_bf16_oracle_against_fused_moe_naive(name):
    """fused_moe_naive runs in fp32 end to end; the native path (and this oracle) round the SiLU
    output to bf16 first, so agreement is to tolerance: relative L2 <= 5e-3."""
    case = cases.bf16_case(name)
    golden = torch.load(os.path.join(GOLDEN, f"bf16_{name}.pt"))["out"].float()
    out = oracle.bf16_forward(case["x"], case["w13"], case["w2"], case["topk_weights"], case["topk_ids"]).float()
    assert float((out - golden).norm() / golden.norm()) <= 5e-3


ACTIVATION_IDS = {"silu": 0, "gelu": 2, "swigluoai": 3}


def oracle_variant(case):
    """The oracle on a BF16 variant case (biases, gelu, swigluoai); interleaved swigluoai weights are reordered to
    gate rows then up rows first, which is what the kernels (and the oracle) take."""
    w13, b13 = case["w13"], case["w13_bias"]
    if case["activation"] == "swigluoai":
        w13 = cases.gate_then_up(w13)
        b13 = None if b13 is None else cases.gate_then_up(b13)
    return oracle.bf16_forward(case["x"], w13, case["w2"], case["topk_weights"], case["topk_ids"], activation=ACTIVATION_IDS[case["activation"]],
                               w13_bias=None if b13 is None else b13.float(), w2_bias=None if case["w2_bias"] is None else case["w2_bias"].float())


@pytest.mark.parametrize("name", sorted(cases.BF16_VARIANTS))
def test_bf16_oracle_variants_against_fused_moe_naive(name):
    """Biases, gelu and swigluoai of the reference's BF16 op: the oracle against fused_moe_naive with the same
    arguments (fp32 end to end there, bf16 intermediate here): relative L2 <= 5e-3."""
    case = cases.bf16_variant_case(name)
    golden = torch.load(os.path.join(GOLDEN, f"bf16_variant_{name}.pt"))["out"].float()
    out = oracle_variant(case).float()
    assert float((out - golden).norm() / golden.norm()) <= 5e-3


@pytest.mark.parametrize("fixed_point", [False, True], ids=["bf16_activations", "fixed_point"])
@pytest.mark.parametrize("name", cases.W8A16_CASES)
def test_w8a16_oracle_against_fused_moe_naive_on_dequantised_weights(name, fixed_point):
    """W8A16 = int8 weights x per-channel scale with 16-bit activations (bf16 as they are, or 16-bit fixed point per
    row with exact integer dot products): the oracle against the reference's fused_moe_naive run on q * scale (fp32):
    relative L2 <= 5e-3."""
    case = cases.w8a8_case(name)
    golden = torch.load(os.path.join(GOLDEN, f"w8a16_{name}.pt"))["out"].float()
    out = oracle.w8a16_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"],
                               fixed_point=fixed_point).float()
    assert float((out - golden).norm() / golden.norm()) <= 5e-3


def test_w8a16_fixed_point_route_rows_track_the_bf16_activation_form():
    """On the fp32 route rows (before any bf16 rounding of the output) the two W8A16 statements differ by the
    fixed-point step of the activations and of the intermediate only."""
    case = cases.w8a8_case("ragged")
    args = (case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"])
    _, plain = oracle.w8a16_forward(*args, dumps=True)
    _, fixed = oracle.w8a16_forward(*args, dumps=True, fixed_point=True)
    difference = float((plain["route_out"] - fixed["route_out"]).norm() / plain["route_out"].norm())
    assert difference <= 1e-3  # measured 2e-4: bf16 roundings of intermediate elements that fall the other way dominate


def test_expneg_tracks_exp():
    for gate in (-20.0, -3.3, -1.0, -1e-3, 0.0, 1e-3, 0.5, 2.0, 9.99, 10.0, 40.0):
        assert oracle.expneg(gate) == pytest.approx(math.exp(-gate), rel=3e-7)


def test_route_build_is_a_stable_sort():
    ids = torch.tensor([[2, 0], [1, 2], [2, 1], [0, 2]], dtype=torch.int64)
    counts, offsets, order = oracle.route_build(ids, 4)
    assert counts.tolist() == [2, 2, 4, 0]
    assert offsets.tolist() == [0, 2, 4, 8, 8]
    assert order.tolist() == [1, 6, 2, 5, 0, 3, 4, 7]
    with pytest.raises(ValueError):
        oracle.route_build(torch.tensor([[4]]), 4)


def test_quantiser_rounding_modes():
    # 2.5/5 -> 0.5*127 = 63.5: a tie.  TORCHREF rounds to even (64), NATIVE away from zero (64); use 62.5.
    row = torch.tensor([[127.0, 62.5, -62.5, 0.5, -0.5, 1.5, 0.0, 0.0] * 2], dtype=torch.bfloat16)
    q_even, s_even = oracle.quantize_rows(row, oracle.NUMERICS_TORCHREF)
    q_away, s_away = oracle.quantize_rows(row, oracle.NUMERICS_NATIVE)
    assert float(s_even[0]) == 1.0 and float(s_away[0]) == 1.0
    assert q_even[0, :6].tolist() == [127, 62, -62, 0, 0, 2]
    assert q_away[0, :6].tolist() == [127, 63, -63, 1, -1, 2]
    zero = torch.zeros((1, 16), dtype=torch.bfloat16)
    assert float(oracle.quantize_rows(zero, oracle.NUMERICS_NATIVE)[1][0]) == 1.0
    assert float(oracle.quantize_rows(zero, oracle.NUMERICS_TORCHREF)[1][0]) == pytest.approx(1e-30)
