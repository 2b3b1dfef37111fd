"""Router front-end (fmoe_router_topk) against torch on the CPU: softmax / sigmoid scoring, top-k, renormalised
weights.  Without a selection bias the kernel selects on the logits (softmax and sigmoid are monotone), so the ids
are EXACTLY torch.topk of the logits; with a bias they must match torch.topk of score + bias wherever two of those
sums are not within rounding of each other.  Weights match to fp32 rounding (rtol 1e-5: the exp implementations
differ in the last place)."""
from __future__ import annotations

import pytest
import torch

from fused_cpp_b200 import _lib, router, synthetic

pytestmark = pytest.mark.gpu

RTOL = 1e-5


def _reference(logits, top_k, scoring, bias, renormalize, scaling):
    scores = torch.softmax(logits, dim=-1) if scoring == "softmax" else torch.sigmoid(logits)
    choice = scores if bias is None else scores + bias
    _, ids = torch.topk(choice, top_k, dim=-1)
    weights = scores.gather(1, ids)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    return weights * scaling, ids, choice


def _check(logits, top_k, scoring="softmax", bias=None, renormalize=True, scaling=1.0):
    device = torch.device("cuda")
    weights, ids = router.router_topk(logits.to(device), top_k, scoring=scoring, selection_bias=None if bias is None else bias.to(device),
                                      renormalize=renormalize, routed_scaling_factor=scaling)
    weights, ids = weights.cpu(), ids.cpu()
    ref_weights, ref_ids, choice = _reference(logits, top_k, scoring, bias, renormalize, scaling)
    assert ids.dtype == torch.int64 and weights.dtype == torch.float32
    if bias is None:
        # Selection on the logits: exactly torch.topk of the logits (distinct values: no tie rule involved).
        assert torch.equal(ids, torch.topk(logits, top_k, dim=-1).indices)
    # Same experts in the same order, except where two reference scores are equal to rounding (then either is right).
    mine = choice.gather(1, ids)
    theirs = choice.gather(1, ref_ids)
    assert torch.allclose(mine, theirs, rtol=4 * RTOL, atol=0.0)
    different = ids != ref_ids
    assert different.float().mean() < 1e-3
    same_rows = ~different.any(dim=1)
    assert torch.allclose(weights[same_rows], ref_weights[same_rows], rtol=RTOL, atol=1e-9)
    assert (ids >= 0).all() and (ids < logits.shape[1]).all()
    # No expert twice in a row.
    assert (torch.sort(ids, dim=1).values.diff(dim=1) != 0).all()


@pytest.mark.parametrize("tokens,experts,top_k", [(1, 256, 8), (16, 16, 4), (64, 256, 8), (333, 257, 6), (8192, 256, 8), (5, 2048, 32),
                                                   (7, 8, 8), (9, 40, 1)])
def test_softmax_topk_matches_torch(cuda_device, tokens, experts, top_k):
    generator = torch.Generator().manual_seed(100 + tokens)
    _check(torch.randn((tokens, experts), generator=generator), top_k)


def test_zipf_biased_logits(cuda_device):
    generator = torch.Generator().manual_seed(5)
    logits = torch.randn((4096, 256), generator=generator) + synthetic.zipf_bias(256, 77)
    _check(logits, 8)


def test_matches_the_benchmark_routing(cuda_device):
    """The benchmark's routing (softmax -> top-8 -> renormalise, synthetic.make_routing) from the same logits."""
    logits = torch.randn((512, 256), generator=torch.Generator().manual_seed(synthetic.SEED_BASE), dtype=torch.float32)
    ref_weights, ref_ids = synthetic.make_routing(512, 256, 8, synthetic.SEED_BASE)
    weights, ids = router.router_topk(logits.cuda(), 8)
    assert (ids.cpu() != ref_ids).float().mean() < 1e-3
    rows = (ids.cpu() == ref_ids).all(dim=1)
    assert torch.allclose(weights.cpu()[rows], ref_weights[rows], rtol=RTOL)


def test_sigmoid_with_selection_bias_and_scaling(cuda_device):
    generator = torch.Generator().manual_seed(9)
    logits = torch.randn((777, 256), generator=generator)
    bias = torch.randn(256, generator=generator) * 0.1
    _check(logits, 8, scoring="sigmoid", bias=bias, renormalize=True, scaling=2.5)
    _check(logits, 8, scoring="sigmoid", bias=None, renormalize=False, scaling=1.0)
    _check(logits, 8, scoring="softmax", bias=bias, renormalize=False, scaling=0.5)


def test_ties_go_to_the_lower_expert(cuda_device):
    logits = torch.zeros((3, 64))
    weights, ids = router.router_topk(logits.cuda(), 4)
    assert ids.cpu().tolist() == [[0, 1, 2, 3]] * 3
    assert torch.allclose(weights.cpu(), torch.full((3, 4), 0.25))


def test_router_feeds_the_forward(cuda_device):
    """Router output goes straight into the W8A8 forward: same result as routing computed by torch on the host."""
    from tests import cases

    case = cases.w8a8_case("tiny")
    device = torch.device("cuda")
    experts = case["w13"].shape[0]
    top_k = case["topk_ids"].shape[1]
    logits = torch.randn((case["x"].shape[0], experts), generator=torch.Generator().manual_seed(3))
    ref_weights, ref_ids, _ = _reference(logits, top_k, "softmax", None, True, 1.0)
    weights, ids = router.router_topk(logits.to(device), top_k)
    assert torch.equal(ids.cpu(), ref_ids)
    c = {k: v.to(device) for k, v in case.items()}
    out = _lib.moe_forward(c["x"], c["w13"], c["w2"], weights, ids, s13=c["s13"], s2=c["s2"]).out
    ref = _lib.moe_forward(c["x"], c["w13"], c["w2"], ref_weights.to(device), ref_ids.to(device), s13=c["s13"], s2=c["s2"]).out
    assert (out.float() - ref.float()).abs().max() <= 2e-2 * ref.float().abs().max()


def test_bad_arguments(cuda_device):
    logits = torch.zeros((2, 8), device="cuda")
    with pytest.raises(ValueError, match="top_k"):
        router.router_topk(logits, 9)
    with pytest.raises(ValueError):
        router.router_topk(logits, 2, scoring="tanh")
    with pytest.raises(ValueError):
        router.router_topk(torch.zeros((2, 8)), 2)
