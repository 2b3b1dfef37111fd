"""Route build on the GPU against the oracle's counting sort (csrc/moe/arm/i8mm_w8a8/kernels.cpp:583-592 restated
in oracle/moe_oracle.c): both forms of the build, the single block used up to 1024 routes and the three kernels
above, at the benchmark's sizes, with Zipf-skewed ids, and with out-of-range ids dropped and reported."""
from __future__ import annotations

import pytest
import torch

from fused_cpp_b200 import _lib, synthetic
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,top_k,skew", [
    (1, 256, 8, False), (64, 256, 8, False), (128, 256, 8, False),   # <= 1024 routes: one block
    (129, 256, 8, False), (700, 256, 8, True), (8192, 256, 8, False), (8192, 256, 8, True), (16384, 257, 8, False),
    (5000, 7, 3, False), (2049, 1, 1, False),
])
def test_route_lists_match_oracle(cuda_device, tokens, experts, top_k, skew):
    if experts >= top_k and experts != 257:
        _, ids = synthetic.make_routing(tokens, experts, top_k, 321 + tokens, skew)
    else:
        ids = torch.randint(0, experts, (tokens, top_k), generator=torch.Generator().manual_seed(tokens), dtype=torch.int64)
    counts, offsets, order = oracle.route_build(ids, experts)
    got_counts, got_offsets, got_order, got_row_expert, status = _lib.route_build_noalloc(ids.to(cuda_device), experts)
    assert status.tolist() == [0, 0]
    assert torch.equal(got_counts.cpu(), counts)
    assert torch.equal(got_offsets.cpu(), offsets)
    assert torch.equal(got_order.cpu(), order)
    assert torch.equal(got_row_expert.cpu().to(torch.int64), ids.reshape(-1)[order.to(torch.int64)])


@pytest.mark.parametrize("tokens", [40, 3000])
def test_bad_ids_are_dropped_and_reported(cuda_device, tokens):
    experts, top_k = 32, 4
    ids = torch.randint(0, experts, (tokens, top_k), generator=torch.Generator().manual_seed(tokens), dtype=torch.int64)
    ids[tokens // 2, 1] = experts + 5
    ids[tokens - 1, 3] = -1
    good = ids.reshape(-1)
    keep = (good >= 0) & (good < experts)
    got_counts, got_offsets, got_order, _, status = _lib.route_build_noalloc(ids.to(cuda_device), experts)
    assert status.tolist()[0] == _lib.ERR_EXPERT_ID_RANGE
    assert status.tolist()[1] in (int((tokens // 2) * top_k + 1), int((tokens - 1) * top_k + 3))
    assert int(got_offsets[-1]) == int(keep.sum())
    expected_counts = torch.bincount(good[keep], minlength=experts).to(torch.int32)
    assert torch.equal(got_counts.cpu(), expected_counts)
    valid = got_order[: int(keep.sum())].cpu().to(torch.int64)
    # stable: inside every expert the flat route ids ascend
    for e in range(experts):
        segment = valid[int(got_offsets[e]): int(got_offsets[e + 1])]
        assert torch.equal(good[segment], torch.full_like(segment, e))
        assert (segment.diff() > 0).all()
