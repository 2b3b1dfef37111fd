"""W8A16 routed-expert MoE on the GPU against the CPU oracle and the golden output of the reference's fused_moe_naive
on the dequantised weights, in both forms of the library: "fixed" (default: activations as 16-bit fixed point per row,
two int8 planes on the int8 tensor cores, exact integer dot products) and "bf16" (activations stay bf16, the int8
weight tiles are widened to bf16 inside the kernel).  Tolerances against the bf16-activation oracle and the golden are
the BF16 path's: relative L2 <= 5e-3, max-abs <= 1e-2 x RMS on the fp32 route rows; the merge is checked exactly on
the GPU's own route rows.  The fixed form is also compared BIT FOR BIT with its own restatement in the oracle
(intermediate rows and fp32 route rows).
"""
from __future__ import annotations

import os

import pytest
import torch

import fused_cpp_b200.moe as moe
from fused_cpp_b200 import _lib, synthetic
from oracle import oracle
from tests import cases
from tests.test_gpu_bf16 import _assert_close_bf16

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


FORMS = {"fixed": _lib.W8A16_FIXED_POINT, "bf16": _lib.W8A16_BF16_ACTIVATIONS}


def _run(case, device, form="fixed", **kw):
    c = {k: v.to(device) for k, v in case.items()}
    return _lib.moe_forward(c["x"], c["w13"], c["w2"], c["topk_weights"], c["topk_ids"], s13=c["s13"], s2=c["s2"], w8a16=True,
                            w8a16_form=FORMS[form], **kw)


def _check_fixed_bit_exact(case, result, limit=0.0):
    """The fixed-point form against fmoe_oracle_w8a16_fixed_forward: integer dot products are exact, so the bf16
    intermediate, the fp32 route rows and the output must agree bit for bit."""
    tokens, hidden = case["x"].shape
    experts, two_i, _ = case["w13"].shape
    top_k = case["topk_ids"].shape[1]
    routes = tokens * top_k
    out_ref, d = oracle.w8a16_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"],
                                      limit, dumps=True, fixed_point=True)
    _, _, order = oracle.route_build(case["topk_ids"], experts)
    y = result.region("y", torch.bfloat16, (routes, two_i // 2)).cpu()
    assert torch.equal(y.view(torch.int16), d["y"][order.long()].view(torch.int16)), "intermediate rows differ from the fixed-point oracle"
    route_out = result.region("route_out", torch.float32, (routes, hidden)).cpu()
    assert torch.equal(route_out.view(torch.int32), d["route_out"].view(torch.int32)), "route rows differ from the fixed-point oracle"
    assert torch.equal(result.out.cpu().view(torch.int16), out_ref.view(torch.int16))


def _check(case, result, limit=0.0, form="bf16"):
    if form == "fixed":
        _check_fixed_bit_exact(case, result, limit)
    assert result.status()[0] == 0
    tokens, hidden = case["x"].shape
    experts, two_i, _ = case["w13"].shape
    top_k = case["topk_ids"].shape[1]
    routes = tokens * top_k
    out_ref, d = oracle.w8a16_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"],
                                      limit, dumps=True)
    _, _, order = oracle.route_build(case["topk_ids"], experts)
    assert torch.equal(result.region("sorted_routes", torch.int32, (routes,)).cpu(), order)
    y = result.region("y", torch.bfloat16, (routes, two_i // 2)).cpu().float()
    y_ref = d["y"][order.long()].float()
    assert float((y - y_ref).norm() / y_ref.norm().clamp_min(1e-30)) <= 5e-3, "activation rows"
    route_out = result.region("route_out", torch.float32, (routes, hidden)).cpu()
    rms = float(d["route_out"].pow(2).mean().sqrt())
    assert float((route_out - d["route_out"]).norm() / d["route_out"].norm()) <= 5e-3
    assert float((route_out - d["route_out"]).abs().max()) <= 1e-2 * rms
    merged = oracle.merge_bf16_path(route_out.view(tokens, top_k, hidden), case["topk_weights"])
    assert torch.equal(result.out.cpu().view(torch.int16), merged.view(torch.int16)), "top-k merge order differs"
    _assert_close_bf16(result.out.cpu(), out_ref, "output vs oracle")


@pytest.mark.parametrize("form", sorted(FORMS))
@pytest.mark.parametrize("tile", [0, 16, 32, 64, 128, 256, 512])
@pytest.mark.parametrize("name", cases.W8A16_CASES)
def test_w8a16_matches_oracle_for_every_row_tile(cuda_device, name, tile, form):
    case = cases.w8a8_case(name)
    _check(case, _run(case, cuda_device, form, gate_up_tile=tile, down_tile=tile), form=form)


@pytest.mark.parametrize("form", sorted(FORMS))
@pytest.mark.parametrize("name", cases.W8A16_CASES)
def test_w8a16_matches_reference_golden(cuda_device, name, form):
    case = cases.w8a8_case(name)
    golden = torch.load(os.path.join(GOLDEN, f"w8a16_{name}.pt"))["out"].float()
    out = _run(case, cuda_device, form).out.cpu().float()
    assert float((out - golden).norm() / golden.norm()) <= 5e-3


@pytest.mark.parametrize("form", sorted(FORMS))
def test_w8a16_clamped_swiglu(cuda_device, form):
    case = cases.w8a8_case("ragged")
    case["x"] = (case["x"].float() * 300).to(torch.bfloat16)  # push gate / up beyond the clamp
    _check(case, _run(case, cuda_device, form, swiglu_limit=10.0), 10.0, form=form)


@pytest.mark.parametrize("form", sorted(FORMS))
@pytest.mark.parametrize("shape", ["decode", "prefill"])
def test_w8a16_at_v3_dims(cuda_device, shape, form):
    """H = 7168, I = 2048 with 8 experts: 112 / 32 K blocks of 64 weights through the widening warps (bf16 form), 56 / 16
    K blocks of 128 against two planes per route (fixed form)."""
    from tests.test_gpu_v3_dims import _w8a8_case

    case = _w8a8_case(shape)
    _check(case, _run(case, cuda_device, form), form=form)


@pytest.mark.parametrize("form", sorted(FORMS))
@pytest.mark.parametrize("activation", [_lib.ACTIVATION_GELU, _lib.ACTIVATION_SWIGLUOAI], ids=["gelu", "swigluoai"])
@pytest.mark.parametrize("name", ["ragged", "wide"])
def test_w8a16_other_activations(cuda_device, name, activation, form):
    """gelu and swigluoai (gate channels then up channels, as the library takes them) through both forms and both
    kernels ("wide" has experts above 64 rows: the two-SM kernel in the fixed form)."""
    case = cases.w8a8_case(name)
    result = _run(case, cuda_device, form, activation=activation)
    assert result.status()[0] == 0
    args = (case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"])
    expected = oracle.w8a16_forward(*args, 0.0, activation=int(activation)).float()
    out = result.out.cpu().float()
    assert float((out - expected).norm() / expected.norm()) <= 5e-3
    if form == "fixed":
        exact = oracle.w8a16_forward(*args, 0.0, activation=int(activation), fixed_point=True)
        # erf / exp of the two sides come from different libraries: the bf16 rounding of the intermediate may differ
        # in the last place on a few elements, so this is a tolerance far below the form's own, not bit-equality.
        assert float((out - exact.float()).norm() / exact.float().norm()) <= 2e-3


def test_w8a16_fixed_point_survives_outliers_and_zero_rows(cuda_device):
    """Rows whose maximum is 2^10 times their typical value (elements far below max / 128 round to the fixed-point
    quantum), an all-zero token and a token of one non-zero element: the fixed form stays bit-exact against its
    restatement and within the tolerance of the bf16-activation oracle."""
    case = cases.w8a8_case("ragged")
    x = case["x"].float()
    x[0].zero_()
    x[1].zero_()
    x[1, 5] = -3.0
    x[2, 7] = 1024.0 * float(x[2].abs().mean())
    x[3, 0] = -1024.0 * float(x[3].abs().mean())
    case["x"] = x.to(torch.bfloat16)
    result = _run(case, cuda_device, "fixed")
    _check_fixed_bit_exact(case, result)
    # Against the bf16-activation statement only the relative L2 is asked here: the outlier rows make intermediate
    # elements of order 1e4, where one bf16 step that falls the other way already moves an output element by more than
    # 1e-2 x RMS, whichever form computed it.
    tokens, hidden = case["x"].shape
    routes = tokens * case["topk_ids"].shape[1]
    _, d = oracle.w8a16_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"], dumps=True)
    route_out = result.region("route_out", torch.float32, (routes, hidden)).cpu()
    assert float((route_out - d["route_out"]).norm() / d["route_out"].norm()) <= 5e-3


@pytest.mark.parametrize("form", sorted(FORMS))
def test_w8a16_repeated_call_is_bit_identical(cuda_device, form):
    case = cases.w8a8_case("wide")
    first = _run(case, cuda_device, form).out.clone()
    second = _run(case, cuda_device, form).out.clone()
    assert torch.equal(first.view(torch.int16), second.view(torch.int16))


def test_w8a16_intermediate_wider_than_hidden(cuda_device):
    """inter > hidden: the planes of the intermediate do not fit the activation-plane region and use their own."""
    generator = torch.Generator().manual_seed(77)
    tokens, hidden, inter, experts, top_k = 24, 64, 160, 4, 2
    case = {
        "x": torch.randn((tokens, hidden), generator=generator).to(torch.bfloat16),
        "w13": torch.randint(-127, 128, (experts, 2 * inter, hidden), generator=generator, dtype=torch.int8),
        "s13": torch.rand((experts, 2 * inter), generator=generator) * 0.002 + 0.0005,
        "w2": torch.randint(-127, 128, (experts, hidden, inter), generator=generator, dtype=torch.int8),
        "s2": torch.rand((experts, hidden), generator=generator) * 0.002 + 0.0005,
        "topk_weights": torch.rand((tokens, top_k), generator=generator),
        "topk_ids": torch.stack([torch.randperm(experts, generator=generator)[:top_k] for _ in range(tokens)]),
    }
    _check(case, _run(case, cuda_device, "fixed"), form="fixed")


def test_w8a16_public_ops(cuda_device):
    """prepare_* (from int8 checkpoint tensors and from bf16), fused_moe_tiled dispatch by weight type under an installed
    runtime, cache_dequant accepted, the routed + shared wrapper, and the rule that W8A16 needs a runtime."""
    shape = cases.W8A8_SHAPES["ragged"]
    case = cases.w8a8_case("ragged")
    x, w, ids = (case[k].to(cuda_device) for k in ("x", "topk_weights", "topk_ids"))
    prepared = moe.prepare_fused_moe_w8a16_tiled_quantized_weights(case["w13"], case["s13"], case["w2"], case["s2"])
    assert isinstance(prepared, moe.PreparedW8A16TiledFusedMoEWeights) and prepared.w13[0].device.type == "cuda"
    previous = moe.set_default_moe_planner_runtime(None)
    try:
        with pytest.raises(RuntimeError, match="requires an installed MoePlannerRuntime"):
            moe.fused_moe_tiled(x, prepared, w, ids)
        runtime = moe.MoePlannerRuntime(None, hidden_size=shape.hidden, intermediate_size=shape.inter, global_experts=shape.experts,
                                        local_experts=shape.experts)
        moe.set_default_moe_planner_runtime(runtime)
        expected = oracle.w8a16_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"])
        for cache_dequant in (False, True):
            out = moe.fused_moe_tiled(x, prepared, w, ids, cache_dequant=cache_dequant)
            _assert_close_bf16(out.cpu(), expected, "fused_moe_tiled(W8A16)")
        assert runtime.last_plan["kind"] == "w8a16"

        # bf16 source weights: quantised per output channel on the GPU, then the same op.
        bf16_case = cases.bf16_case("top8")
        from_bf16 = moe.prepare_fused_moe_w8a16_tiled_weights(bf16_case["w13"], bf16_case["w2"])
        q13, s13 = from_bf16.w13[0].cpu(), from_bf16.w13[3].cpu()
        q2, s2 = from_bf16.w2[0].cpu(), from_bf16.w2[3].cpu()
        top8 = cases.BF16_SHAPES["top8"]
        moe.set_default_moe_planner_runtime(moe.MoePlannerRuntime(None, hidden_size=top8.hidden, intermediate_size=top8.inter,
                                                                  global_experts=top8.experts, local_experts=top8.experts))
        out = moe.fused_moe_w8a16_tiled(bf16_case["x"].to(cuda_device), from_bf16, bf16_case["topk_weights"].to(cuda_device),
                                        bf16_case["topk_ids"].to(cuda_device))
        expected = oracle.w8a16_forward(bf16_case["x"], q13, s13, q2, s2, bf16_case["topk_weights"], bf16_case["topk_ids"])
        _assert_close_bf16(out.cpu(), expected, "W8A16 from bf16 weights")

        # routed + shared
        sw13, ss13, sw2, ss2 = synthetic.make_int8_expert(shape.hidden, shape.inter, 424242)
        shared = moe.prepare_routed_shared_moe_w8a16_tiled_quantized_weights(case["w13"], case["s13"], case["w2"], case["s2"],
                                                                             sw13, ss13, sw2, ss2)
        moe.set_default_moe_planner_runtime(moe.MoePlannerRuntime(None, hidden_size=shape.hidden, intermediate_size=shape.inter,
                                                                  global_experts=shape.experts, local_experts=shape.experts, shared_experts=1))
        out = moe.fused_moe_w8a16_tiled_with_shared(x, shared, w, ids, routed_scaling_factor=2.5)
        tokens = shape.tokens
        all_ids = torch.cat((case["topk_ids"], torch.full((tokens, 1), shape.experts, dtype=torch.int64)), 1)
        all_w = torch.cat((case["topk_weights"] * 2.5, torch.ones((tokens, 1))), 1)
        expected = oracle.w8a16_forward(case["x"], torch.cat((case["w13"], sw13[None]), 0), torch.cat((case["s13"], ss13[None]), 0),
                                        torch.cat((case["w2"], sw2[None]), 0), torch.cat((case["s2"], ss2[None]), 0), all_w, all_ids)
        _assert_close_bf16(out.cpu(), expected, "W8A16 routed + shared")
    finally:
        moe.set_default_moe_planner_runtime(previous)
