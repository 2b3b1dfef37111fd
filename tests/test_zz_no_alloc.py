"""The allocation-free route build (fmoe_route_build_noalloc) against the regular forward's route lists.

This entry point is for hosts that cannot allocate device memory while they serve (all of HBM already
belongs to a KV-cache pool, or the memory plan is frozen after warm-up): its scratch is a fixed array
inside the library instead of a caller workspace.  The file name keeps it last in collection order, so a
run that stops at the first failure has already exercised every other test.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from fused_cpp_b200 import _lib
from tests import cases

pytestmark = pytest.mark.gpu


def _reference_lists(case, device):
    """Route lists as the existing entry point (fmoe_w8a8_forward) leaves them in its workspace."""
    cuda = {k: v.to(device) for k, v in case.items()}
    result = _lib.moe_forward(cuda["x"], cuda["w13"], cuda["w2"], cuda["topk_weights"], cuda["topk_ids"], s13=cuda["s13"], s2=cuda["s2"])
    assert result.status()[0] == 0
    experts = case["w13"].shape[0]
    routes = case["topk_ids"].numel()
    return (result.region("counts", torch.int32, (experts,)).clone(), result.region("offsets", torch.int32, (experts + 1,)).clone(),
            result.region("sorted_routes", torch.int32, (routes,)).clone(), result.region("row_expert", torch.int32, (routes,)).clone())


def test_noalloc_route_build_matches_forward_twice_in_a_row(cuda_device):
    # Two calls in a row on different problems: the second is smaller and has an expert without routes, so
    # anything the first call left in the shared scratch would show up as a wrong count or position.
    for name in ("wide", "ragged"):
        case = cases.w8a8_case(name)
        expected = _reference_lists(case, cuda_device)
        experts = case["w13"].shape[0]
        counts, offsets, order, row_expert, status = _lib.route_build_noalloc(case["topk_ids"].to(cuda_device), experts)
        assert status.tolist() == [0, 0]
        for got, want, what in zip((counts, offsets, order, row_expert), expected, ("counts", "offsets", "sorted_routes", "row_expert")):
            assert torch.equal(got, want), f"{name}: {what} differs from the forward call's route lists"


def test_noalloc_reports_bad_ids_and_refuses_oversize(cuda_device):
    ids = cases.w8a8_case("tiny")["topk_ids"].clone()
    ids[1, 0] = -3
    *_, status = _lib.route_build_noalloc(ids.to(cuda_device), 4)
    assert status.tolist() == [_lib.ERR_EXPERT_ID_RANGE, 2]
    # and the next call starts from a clean status block again
    *_, status = _lib.route_build_noalloc(cases.w8a8_case("tiny")["topk_ids"].to(cuda_device), 4)
    assert status.tolist() == [0, 0]
    too_many = torch.zeros((131072 // 8 + 1, 8), dtype=torch.int64, device=cuda_device)
    with pytest.raises(ValueError, match="exceeds the static scratch"):
        _lib.route_build_noalloc(too_many, 16)
    with pytest.raises(ValueError, match="exceeds the static scratch"):
        _lib.route_build_noalloc(torch.zeros((4, 2), dtype=torch.int64, device=cuda_device), 513)


def test_noalloc_call_leaves_the_allocator_alone(cuda_device):
    """Raw C-ABI call with pre-made outputs: torch's allocator statistics do not move across it."""
    case = cases.w8a8_case("wide")
    ids = case["topk_ids"].to(cuda_device)
    experts = case["w13"].shape[0]
    routes = ids.numel()
    outs = [torch.empty(n, dtype=torch.int32, device=cuda_device) for n in (experts, experts + 1, routes, routes, 2)]
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"], torch.cuda.memory_reserved()
    lib = _lib.load()
    code = lib.fmoe_route_build_noalloc(ctypes.c_void_p(ids.data_ptr()), ids.shape[0], ids.shape[1], experts,
                                        *[ctypes.c_void_p(t.data_ptr()) for t in outs],
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert code == 0
    after = torch.cuda.memory_stats()["allocation.all.allocated"], torch.cuda.memory_reserved()
    assert before == after
    assert outs[4].tolist() == [0, 0] and int(outs[1][-1]) == routes
