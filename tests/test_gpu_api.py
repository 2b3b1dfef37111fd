"""The public fused_cpp-style API on the GPU: prepare_*, fused_moe_tiled, routed+shared wrappers, out=,
weight quantiser.  Parity is against the CPU oracle (bit-exact for W8A8)."""
from __future__ import annotations

import os

import pytest
import torch

import fused_cpp_b200.moe as moe
from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu


@pytest.fixture()
def runtime_for():
    installed = []

    def install(shape, shared=0):
        runtime = moe.MoePlannerRuntime(None, hidden_size=shape.hidden, intermediate_size=shape.inter,
                                        global_experts=shape.experts, local_experts=shape.experts, shared_experts=shared)
        installed.append(moe.set_default_moe_planner_runtime(runtime))
        return runtime

    yield install
    moe.set_default_moe_planner_runtime(installed[0] if installed else None)


def test_w8a8_public_path_matches_oracle(cuda_device, runtime_for):
    name = "ragged"
    case = cases.w8a8_case(name)
    runtime = runtime_for(cases.W8A8_SHAPES[name])
    weights = moe.prepare_fused_moe_w8a8_tiled_quantized_weights(case["w13"], case["s13"], case["w2"], case["s2"])
    assert weights.w13[0].device.type == "cuda"
    out = moe.fused_moe_tiled(case["x"].to(cuda_device), weights, case["topk_weights"].to(cuda_device),
                              case["topk_ids"].to(cuda_device), swiglu_limit=10.0)
    expected = oracle.w8a8_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"])
    assert torch.equal(out.cpu().view(torch.int16), expected.view(torch.int16))
    assert runtime.last_plan["kind"] == "int8"
    with pytest.raises(ValueError, match="swiglu_limit=10.0"):
        moe.fused_moe_tiled(case["x"].to(cuda_device), weights, case["topk_weights"].to(cuda_device),
                            case["topk_ids"].to(cuda_device), swiglu_limit=0.0)


def test_out_buffer_is_written_in_place_and_returned(cuda_device, runtime_for):
    case = cases.w8a8_case("tiny")
    runtime_for(cases.W8A8_SHAPES["tiny"])
    weights = moe.prepare_fused_moe_w8a8_tiled_quantized_weights(case["w13"], case["s13"], case["w2"], case["s2"])
    x = case["x"].to(cuda_device)
    out = torch.full_like(x, 7.0)
    returned = moe.fused_moe_tiled(x, weights, case["topk_weights"].to(cuda_device), case["topk_ids"].to(cuda_device),
                                   swiglu_limit=10.0, out=out)
    assert returned is out
    expected = oracle.w8a8_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"])
    assert torch.equal(out.cpu().view(torch.int16), expected.view(torch.int16))
    with pytest.raises(ValueError, match="out must"):
        moe.fused_moe_tiled(x, weights, case["topk_weights"].to(cuda_device), case["topk_ids"].to(cuda_device),
                            swiglu_limit=10.0, out=torch.empty((3, 3), dtype=torch.bfloat16, device=cuda_device))


def test_bf16_weight_quantiser_matches_explicit_channel_quantisation(cuda_device):
    """prepare(bf16) == prepare(pre-quantised), the reference's tests/test_moe_w8a8.py:233-251."""
    generator = torch.Generator().manual_seed(29)
    w13 = (torch.randn((2, 32, 16), generator=generator) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn((2, 16, 16), generator=generator) * 0.1).to(torch.bfloat16)
    w13[1, 5].zero_()

    def quantize(weight):
        fp32 = weight.float()
        maximum = fp32.abs().amax(dim=-1, keepdim=True)
        scale = torch.where(maximum > 0, maximum / 127.0, torch.ones_like(maximum))
        return (fp32 / scale).round().clamp(-127, 127).to(torch.int8), scale.squeeze(-1)

    q13, s13 = quantize(w13)
    q2, s2 = quantize(w2)
    automatic = moe.prepare_fused_moe_w8a8_tiled_weights(w13, w2)
    assert torch.equal(automatic.w13[0].cpu(), q13) and torch.equal(automatic.w13[3].cpu(), s13)
    assert torch.equal(automatic.w2[0].cpu(), q2) and torch.equal(automatic.w2[3].cpu(), s2)


def test_w8a8_routed_plus_shared_equals_explicit_concatenation(cuda_device, runtime_for):
    """The shared expert is expert id E appended as route K with weight 1 (bf16_tiled.py:1007-1013 of the reference)."""
    shape = cases.W8A8_SHAPES["ragged"]
    case = cases.w8a8_case("ragged")
    runtime_for(shape, shared=1)
    from fused_cpp_b200 import synthetic
    sw13, ss13, sw2, ss2 = synthetic.make_int8_expert(shape.hidden, shape.inter, 424242)
    weights = moe.prepare_routed_shared_moe_w8a8_tiled_quantized_weights(case["w13"], case["s13"], case["w2"], case["s2"],
                                                                         sw13, ss13, sw2, ss2)
    assert weights.shared_expert_id == shape.experts and weights.packed.w13[0].shape[0] == shape.experts + 1
    out = moe.fused_moe_w8a8_tiled_with_shared(case["x"].to(cuda_device), weights, case["topk_weights"].to(cuda_device),
                                               case["topk_ids"].to(cuda_device), routed_scaling_factor=2.5)
    tokens = shape.tokens
    ids = torch.cat((case["topk_ids"], torch.full((tokens, 1), shape.experts, dtype=torch.int64)), 1)
    w = torch.cat((case["topk_weights"] * 2.5, torch.ones((tokens, 1))), 1)
    expected = oracle.w8a8_forward(case["x"], torch.cat((case["w13"], sw13[None]), 0), torch.cat((case["s13"], ss13[None]), 0),
                                   torch.cat((case["w2"], sw2[None]), 0), torch.cat((case["s2"], ss2[None]), 0), w, ids)
    assert torch.equal(out.cpu().view(torch.int16), expected.view(torch.int16))


def test_bf16_public_path_and_shared_mlp(cuda_device):
    case = cases.bf16_case("top8")
    weights = moe.prepare_fused_moe_bf16_tiled_weights(case["w13"], case["w2"], fuse_silu=True)
    assert weights.backend_name == "cuda_sm100_tcgen05" and moe.available_fused_moe_bf16_tiled_backends() == ("cuda_sm100_tcgen05",)
    out = moe.fused_moe_bf16_tiled(case["x"].to(cuda_device), weights, case["topk_weights"].to(cuda_device),
                                   case["topk_ids"].to(torch.int32).to(cuda_device))
    expected = oracle.bf16_forward(case["x"], case["w13"], case["w2"], case["topk_weights"], case["topk_ids"])
    assert float((out.cpu().float() - expected.float()).norm() / expected.float().norm()) <= 5e-3
    shared = moe.prepare_shared_mlp_bf16_tiled_weights(case["w13"][0], case["w2"][0])
    mlp = moe.shared_mlp_bf16_tiled(case["x"].to(cuda_device), shared)
    ones = torch.ones((case["x"].shape[0], 1))
    zeros = torch.zeros((case["x"].shape[0], 1), dtype=torch.int64)
    mlp_ref = oracle.bf16_forward(case["x"], case["w13"][:1], case["w2"][:1], ones, zeros)
    assert float((mlp.cpu().float() - mlp_ref.float()).norm() / mlp_ref.float().norm()) <= 5e-3


def test_forward_rejects_cpu_tensors(cuda_device):
    case = cases.bf16_case("tiny")
    weights = moe.prepare_fused_moe_bf16_tiled_weights(case["w13"], case["w2"])
    # The device rule belongs to the native op (a TORCH_CHECK-style RuntimeError), not to the Python wrapper.
    with pytest.raises(RuntimeError, match="CUDA"):
        moe.fused_moe_bf16_tiled(case["x"], weights, case["topk_weights"], case["topk_ids"])


@pytest.mark.parametrize("tile", [0, 512], ids=["auto", "two_sm"])
@pytest.mark.parametrize("name", sorted(cases.BF16_VARIANTS))
def test_bf16_op_biases_gelu_and_swigluoai(cuda_device, name, tile):
    """w13_bias / w2_bias and the gelu / swigluoai activations of the reference's BF16 op
    (csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:6420-6427, :1911-1936) against the oracle and against the golden
    output of fused_moe_naive with the same arguments; swigluoai weights arrive interleaved, as in a checkpoint."""
    from tests.test_oracle_golden import oracle_variant

    case = cases.bf16_variant_case(name)
    prepared = moe.prepare_fused_moe_bf16_tiled_weights(case["w13"], case["w2"], fuse_silu=True)
    plan = moe.plan.gpu_placeholder_plan(tile, tile)
    out = moe.fused_moe_bf16_tiled_async_plan(case["x"].to(cuda_device), prepared, case["topk_weights"].to(cuda_device),
                                              case["topk_ids"].to(cuda_device), plan, w13_bias=case["w13_bias"], w2_bias=case["w2_bias"],
                                              activation=case["activation"]).cpu().float()
    expected = oracle_variant(case).float()
    assert float((out - expected).norm() / expected.norm()) <= 5e-3
    golden = torch.load(os.path.join(os.path.dirname(__file__), "golden", f"bf16_variant_{name}.pt"))["out"].float()
    assert float((out - golden).norm() / golden.norm()) <= 5e-3


def test_bf16_op_global_num_experts_narrows_the_valid_ids(cuda_device):
    """global_num_experts below the prepared expert count makes the ids beyond it invalid, as in the reference
    (fused_moe_bf16_tiled.cpp:6439-6458), instead of routing them to the trailing experts."""
    case = cases.bf16_case("top8")  # 16 experts
    prepared = moe.prepare_fused_moe_bf16_tiled_weights(case["w13"], case["w2"], fuse_silu=True)
    x, w, ids = (case[k].to(cuda_device) for k in ("x", "topk_weights", "topk_ids"))
    assert int(ids.max()) >= 12
    with pytest.raises(Exception, match="out of range"):
        moe.fused_moe_bf16_tiled(x, prepared, w, ids, global_num_experts=12)
    full = moe.fused_moe_bf16_tiled(x, prepared, w, ids, global_num_experts=16)
    assert torch.equal(full, moe.fused_moe_bf16_tiled(x, prepared, w, ids))
