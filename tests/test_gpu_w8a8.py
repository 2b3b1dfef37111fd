"""W8A8 routed-expert MoE on the GPU, through the C ABI, against the CPU oracle and the golden
outputs of the reference's own Python functions.  Integer and byte results are compared bit-exactly;
so are the bf16/fp32 stages, because the kernels follow the reference's arithmetic step by step
with IEEE operations (tolerance 0 everywhere in this file).
"""
from __future__ import annotations

import os

import pytest
import torch

from fused_cpp_b200 import _lib, synthetic
from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
IMPLS = {"simt": _lib.GEMM_SIMT, "umma": _lib.GEMM_UMMA}


def _to_cuda(case, device):
    return {k: v.to(device) for k, v in case.items()}


def _run(case, device, **kw):
    c = _to_cuda(case, device)
    return _lib.moe_forward(c["x"], c["w13"], c["w2"], c["topk_weights"], c["topk_ids"], s13=c["s13"], s2=c["s2"], **kw)


def _check_all_stages(case, result, numerics):
    tokens, hidden = case["x"].shape
    experts, two_i, _ = case["w13"].shape
    inter = two_i // 2
    top_k = case["topk_ids"].shape[1]
    routes = tokens * top_k
    out_ref, d = oracle.w8a8_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"],
                                     case["topk_ids"], numerics, dumps=True)
    counts_ref, offsets_ref, order_ref = oracle.route_build(case["topk_ids"], experts)
    error, detail = result.status()
    assert error == 0, (error, detail)
    order = result.region("sorted_routes", torch.int32, (routes,)).cpu()
    assert torch.equal(result.region("counts", torch.int32, (experts,)).cpu(), counts_ref)
    assert torch.equal(result.region("offsets", torch.int32, (experts + 1,)).cpu(), offsets_ref)
    assert torch.equal(order, order_ref), "route lists differ"
    assert torch.equal(result.region("row_expert", torch.int32, (routes,)).cpu().long(),
                       case["topk_ids"].reshape(-1)[order.long()])
    token_of_row = (order // top_k).long()
    flat = order.long()
    route_pos = result.region("route_pos", torch.int32, (routes,)).cpu().long()
    assert torch.equal(route_pos[flat], torch.arange(routes)), "route_pos is not the inverse of sorted_routes"
    assert torch.equal(result.region("a_rows", torch.int8, (routes, hidden)).cpu(), d["xq"][token_of_row]), "xq differs"
    assert torch.equal(result.region("a_scale", torch.float32, (routes,)).cpu(), d["a"][token_of_row]), "a differs"
    assert torch.equal(result.acc1.cpu(), d["acc1"][flat]), "gate_up int32 accumulators differ"
    y = result.region("y", torch.bfloat16, (routes, inter)).cpu()
    assert torch.equal(y.view(torch.int16), d["y"][flat].view(torch.int16)), "SwiGLU output differs"
    assert torch.equal(result.region("yq", torch.int8, (routes, inter)).cpu(), d["yq"][flat]), "yq differs"
    assert torch.equal(result.region("y_scale", torch.float32, (routes,)).cpu(), d["a2"][flat]), "a2 differs"
    assert torch.equal(result.acc2.cpu(), d["acc2"][flat]), "down int32 accumulators differ"
    route_out = result.region("route_out", torch.float32, (routes, hidden)).cpu()
    assert torch.equal(route_out, d["route_out"]), "route_out differs"
    assert torch.equal(result.out.cpu().view(torch.int16), out_ref.view(torch.int16)), "output differs"


@pytest.mark.parametrize("impl", ["simt", "umma"])
@pytest.mark.parametrize("numerics", [0, 1], ids=["torchref", "native"])
@pytest.mark.parametrize("name", cases.W8A8_CASES)
def test_w8a8_every_stage_matches_oracle(cuda_device, name, numerics, impl):
    case = cases.w8a8_case(name)
    result = _run(case, cuda_device, numerics=numerics, gemm_impl=IMPLS[impl], dump=True)
    _check_all_stages(case, result, numerics)


@pytest.mark.parametrize("impl", ["simt", "umma"])
@pytest.mark.parametrize("name", cases.W8A8_CASES)
def test_w8a8_matches_reference_golden(cuda_device, name, impl):
    """Golden = tests/test_moe_w8a8.py::_quantize_row/_reference of the reference, run on the same inputs."""
    case = cases.w8a8_case(name)
    golden = torch.load(os.path.join(GOLDEN, f"w8a8_{name}.pt"))
    result = _run(case, cuda_device, numerics=_lib.NUMERICS_TORCHREF, gemm_impl=IMPLS[impl])
    top_k = case["topk_ids"].shape[1]
    routes = case["topk_ids"].numel()
    hidden = case["x"].shape[1]
    order = result.region("sorted_routes", torch.int32, (routes,)).cpu()
    token_of_row = (order // top_k).long()
    assert torch.equal(result.region("a_rows", torch.int8, (routes, hidden)).cpu(), golden["xq"][token_of_row])
    assert torch.equal(result.region("a_scale", torch.float32, (routes,)).cpu(), golden["a"].float()[token_of_row])
    # The reference's own native-vs-Python tolerance is atol=3e-6 (tests/test_moe_w8a8.py:225); this path is bit-exact.
    assert torch.equal(result.out.cpu().view(torch.int16), golden["out"].view(torch.int16))


def _skewed_case(tokens=300, experts=14, top_k=3, hidden=128, inter=96):
    """One expert takes a route of every token (hundreds of rows), one takes 70, the rest a handful, one none:
    with automatic tiles the experts above 64 rows go to the two-SM kernel and the others to the one-SM kernel
    in the same forward."""
    shape = synthetic.MoEShape(tokens=tokens, hidden=hidden, inter=inter, experts=experts, top_k=top_k)
    case = synthetic.make_w8a8_case(shape, seed=424242)
    generator = torch.Generator().manual_seed(99)
    ids = torch.empty((tokens, top_k), dtype=torch.int64)
    ids[:, 0] = 0
    ids[:, 1] = torch.where(torch.arange(tokens) < 70, torch.full((tokens,), 1), 2 + torch.randint(0, 5, (tokens,), generator=generator))
    ids[:, 2] = 7 + torch.randint(0, 6, (tokens,), generator=generator)  # experts 7..12; expert 13 stays empty
    case["topk_ids"] = ids
    return case


@pytest.mark.parametrize("numerics", [0, 1], ids=["torchref", "native"])
def test_w8a8_experts_split_between_the_two_kernels(cuda_device, numerics):
    case = _skewed_case()
    counts = torch.bincount(case["topk_ids"].reshape(-1), minlength=14)
    assert counts.max() > 256 and (counts > 64).sum() >= 2 and ((counts > 0) & (counts <= 64)).sum() >= 5 and counts[13] == 0
    result = _run(case, cuda_device, numerics=numerics, gemm_impl=_lib.GEMM_UMMA, dump=True)
    _check_all_stages(case, result, numerics)
    assert result.status_word(6) > 0 and result.status_word(2) > 0  # both kernels had work items


@pytest.mark.parametrize("name", ["wide", "cfg1", "ragged"])
def test_w8a8_two_sm_pair_kernel_matches_oracle(cuda_device, name):
    """Row tile 512 selects the cta_group::2 kernel (256-row work items, a cluster of two CTAs per tile)."""
    case = cases.w8a8_case(name)
    result = _run(case, cuda_device, gemm_impl=_lib.GEMM_UMMA, gate_up_tile=512, down_tile=512, dump=True)
    _check_all_stages(case, result, 0)


@pytest.mark.parametrize("tile", [16, 32, 64, 128, 256])
def test_w8a8_row_tile_does_not_change_results(cuda_device, tile):
    """Every row-tile configuration of the tcgen05 kernel gives the same bits (the reference's
    route-slice tests, tests/test_fused_moe_bf16_tiled.py:358-464, recast for tile height)."""
    case = cases.w8a8_case("wide")
    result = _run(case, cuda_device, gemm_impl=_lib.GEMM_UMMA, gate_up_tile=tile, down_tile=tile, dump=True)
    _check_all_stages(case, result, 0)


def test_w8a8_more_than_65535_tokens(cuda_device):
    """The reference accepts any token count; the merge must not put tokens on a 65535-limited grid axis."""
    shape = synthetic.MoEShape(tokens=70000, hidden=64, inter=64, experts=2, top_k=2)
    case = synthetic.make_w8a8_case(shape, seed=31337)
    result = _run(case, cuda_device, dump=True)
    _check_all_stages(case, result, 0)


@pytest.mark.parametrize("name", ["cfg1", "wide", "ragged"])
def test_w8a8_compact_route_rows_keep_the_integer_stages_exact(cuda_device, name):
    """route_rows_bf16 (opt-in): the down GEMM stores bf16 rows.  Everything up to and including the int32 down
    accumulators stays bit-exact; the stored rows are the bf16 rounding of the exact fp32 rows; the output is the
    reference's fma chain over those rounded rows (exactly), hence within tolerance of the fp32-row result."""
    case = cases.w8a8_case(name)
    result = _run(case, cuda_device, dump=True, route_rows_bf16=True)
    assert result.status()[0] == 0
    tokens, hidden = case["x"].shape
    top_k = case["topk_ids"].shape[1]
    routes = tokens * top_k
    out_ref, d = oracle.w8a8_forward(case["x"], case["w13"], case["s13"], case["w2"], case["s2"], case["topk_weights"], case["topk_ids"], 0,
                                     dumps=True)
    order = result.region("sorted_routes", torch.int32, (routes,)).cpu().long()
    assert torch.equal(result.acc1.cpu(), d["acc1"][order]) and torch.equal(result.acc2.cpu(), d["acc2"][order])
    assert torch.equal(result.region("yq", torch.int8, (routes, case["w13"].shape[1] // 2)).cpu(), d["yq"][order])
    rows = result.region("route_out", torch.bfloat16, (routes, hidden)).cpu()
    assert torch.equal(rows.view(torch.int16), d["route_out"].to(torch.bfloat16).view(torch.int16)), "rows are not the rounded exact rows"
    merged = oracle.merge_w8a8_path(rows.float().view(tokens, top_k, hidden), case["topk_weights"])
    assert torch.equal(result.out.cpu().view(torch.int16), merged.view(torch.int16))
    error = (result.out.cpu().float() - out_ref.float()).norm() / out_ref.float().norm()
    assert float(error) <= 5e-3


def test_w8a8_repeated_call_is_bit_identical(cuda_device):
    case = cases.w8a8_case("ragged")
    first = _run(case, cuda_device).out.clone()
    second = _run(case, cuda_device).out.clone()
    assert torch.equal(first.view(torch.int16), second.view(torch.int16))


def test_w8a8_identical_rows_give_identical_outputs(cuda_device):
    """A token's result does not depend on its position in the batch (docs/public_contracts.md:38-42)."""
    case = cases.w8a8_case("wide")
    case["x"][57] = case["x"][3]
    case["topk_ids"][57] = case["topk_ids"][3]
    case["topk_weights"][57] = case["topk_weights"][3]
    out = _run(case, cuda_device).out.cpu()
    assert torch.equal(out[57].view(torch.int16), out[3].view(torch.int16))


def test_w8a8_out_of_range_expert_id_is_reported(cuda_device):
    case = cases.w8a8_case("tiny")
    case["topk_ids"][2, 1] = 99
    result = _run(case, cuda_device)
    error, detail = result.status()
    assert error == _lib.ERR_EXPERT_ID_RANGE and detail == 2 * case["topk_ids"].shape[1] + 1
    with pytest.raises(_lib.FusedMoEError, match="out of range"):
        result.raise_for_status()


def test_w8a8_rejects_unclamped_activation(cuda_device):
    case = cases.w8a8_case("tiny")
    with pytest.raises(ValueError, match="limit 10.0"):
        _run(case, cuda_device, swiglu_limit=0.0)


def test_w8a8_empty_batch(cuda_device):
    case = cases.w8a8_case("tiny")
    case["x"] = case["x"][:0]
    case["topk_ids"] = case["topk_ids"][:0]
    case["topk_weights"] = case["topk_weights"][:0]
    assert _run(case, cuda_device).out.shape == (0, 64)


def test_row_quantiser_hook_matches_oracle(cuda_device):
    x = cases.w8a8_case("cfg1")["x"]
    for numerics in (0, 1):
        q, scale = _lib.quantize_rows(x.to(cuda_device), numerics)
        q_ref, scale_ref = oracle.quantize_rows(x, numerics)
        assert torch.equal(q.cpu(), q_ref) and torch.equal(scale.cpu(), scale_ref)
