"""Parity at the dimensions the benchmark runs at: H=7168, I=2048 (DeepSeek-V3-scale experts).

The small cases elsewhere in tests/ never reach K=7168 (56 K-blocks of 128 bytes, int32 sums up to 1.2e8),
I=2048 through the two-SM kernel's 5-D weight map, or several 256-row work items per expert at full width.
Here the expert count is reduced to 8 so that the CPU oracle finishes in seconds; everything per expert and
per route is the benchmark's.  Two shapes per path:

  decode   T=64, top-2, near-uniform routing: every expert holds at most 64 rows, so the one-SM kernel
           with its 64-row tile does all the work (the decode regime of the benchmark);
  prefill  T=600, top-4, Zipf-biased routing (seed chosen so that two experts exceed 512 rows, two more exceed
           256, three sit between 65 and 256 and one stays below 64): with automatic tiles the device-side
           split sends the thin expert to the one-SM kernel and the others to the two-SM kernel with one, two
           or three work items per expert; a second run forces every expert through the two-SM kernel.

W8A8 is compared bit for bit at every stage (routes, int8 rows, scales, int32 accumulators, bf16 intermediate,
requantised rows, fp32 route rows, bf16 output); BF16 at the tolerances of tests/test_gpu_bf16.py.
The input recipe is the benchmark's (fused_cpp_b200.synthetic), which is the reference's seed-23 recipe
(tests/test_moe_w8a8.py:201-226) with the benchmark's value ranges.
"""
from __future__ import annotations

import functools

import pytest
import torch

from fused_cpp_b200 import _lib, synthetic
from oracle import oracle
from tests.test_gpu_bf16 import _assert_close_bf16
from tests.test_gpu_w8a8 import _check_all_stages

pytestmark = pytest.mark.gpu

HIDDEN, INTER, EXPERTS = 7168, 2048, 8
SHAPES = {
    "decode": (synthetic.MoEShape(tokens=64, hidden=HIDDEN, inter=INTER, experts=EXPERTS, top_k=2), 555, False),
    "prefill": (synthetic.MoEShape(tokens=600, hidden=HIDDEN, inter=INTER, experts=EXPERTS, top_k=4), 777, True),
}


@functools.lru_cache(maxsize=None)
def _w8a8_weights():
    return synthetic.make_int8_weights(SHAPES["decode"][0], seed=synthetic.SEED_BASE + 90000)


@functools.lru_cache(maxsize=None)
def _bf16_weights():
    return synthetic.make_bf16_weights(SHAPES["decode"][0], seed=synthetic.SEED_BASE + 91000)


def _batch(name: str) -> dict:
    shape, seed, skew = SHAPES[name]
    topk_w, topk_ids = synthetic.make_routing(shape.tokens, shape.experts, shape.top_k, seed, skew)
    return {"x": synthetic.make_activations(shape.tokens, shape.hidden, seed + 1), "topk_weights": topk_w, "topk_ids": topk_ids}


def _w8a8_case(name: str) -> dict:
    w13, s13, w2, s2 = _w8a8_weights()
    return {**_batch(name), "w13": w13, "s13": s13, "w2": w2, "s2": s2}


def _bf16_case(name: str) -> dict:
    w13, w2 = _bf16_weights()
    return {**_batch(name), "w13": w13, "w2": w2}


def _run(case, device, **kw):
    c = {k: v.to(device) for k, v in case.items()}
    scales = {"s13": c["s13"], "s2": c["s2"]} if "s13" in c else {}
    return _lib.moe_forward(c["x"], c["w13"], c["w2"], c["topk_weights"], c["topk_ids"], **scales, **kw)


def test_prefill_routing_exercises_every_item_count():
    counts = torch.bincount(_batch("prefill")["topk_ids"].reshape(-1), minlength=EXPERTS)
    assert (counts > 512).sum() >= 1, counts
    assert ((counts > 256) & (counts <= 512)).sum() >= 1, counts
    assert ((counts > 64) & (counts <= 256)).sum() >= 2, counts
    assert ((counts > 0) & (counts <= 64)).sum() >= 1, counts
    assert int(torch.bincount(_batch("decode")["topk_ids"].reshape(-1), minlength=EXPERTS).max()) <= 64


@pytest.mark.parametrize("numerics", [0, 1], ids=["torchref", "native"])
def test_w8a8_decode_tile_at_v3_dims(cuda_device, numerics):
    case = _w8a8_case("decode")
    result = _run(case, cuda_device, numerics=numerics, dump=True)
    _check_all_stages(case, result, numerics)
    assert result.status_word(2) > 0 and result.status_word(6) == 0  # one-SM kernel only


@pytest.mark.parametrize("tiles", [(0, 0), (512, 512)], ids=["device_split", "two_sm_only"])
def test_w8a8_prefill_kernels_at_v3_dims(cuda_device, tiles):
    case = _w8a8_case("prefill")
    result = _run(case, cuda_device, gate_up_tile=tiles[0], down_tile=tiles[1], dump=True)
    _check_all_stages(case, result, 0)
    if tiles == (0, 0):
        assert result.status_word(2) > 0 and result.status_word(6) > 0  # both kernels had work items


def test_w8a8_prefill_native_numerics_at_v3_dims(cuda_device):
    case = _w8a8_case("prefill")
    result = _run(case, cuda_device, numerics=1, dump=True)
    _check_all_stages(case, result, 1)


@pytest.mark.parametrize("tiles", [(0, 0), (512, 512)], ids=["auto", "two_sm_only"])
@pytest.mark.parametrize("name", ["decode", "prefill"])
def test_bf16_at_v3_dims(cuda_device, name, tiles):
    case = _bf16_case(name)
    result = _run(case, cuda_device, gate_up_tile=tiles[0], down_tile=tiles[1])
    assert result.status()[0] == 0
    tokens, hidden = case["x"].shape
    top_k = case["topk_ids"].shape[1]
    routes = tokens * top_k
    out_ref, d = oracle.bf16_forward(case["x"], case["w13"], case["w2"], case["topk_weights"], case["topk_ids"], 0.0, dumps=True)
    _, _, order = oracle.route_build(case["topk_ids"], EXPERTS)
    assert torch.equal(result.region("sorted_routes", torch.int32, (routes,)).cpu(), order)
    y = result.region("y", torch.bfloat16, (routes, INTER)).cpu().float()
    y_ref = d["y"][order.long()].float()
    assert float((y - y_ref).norm() / y_ref.norm()) <= 5e-3, "SiLU(gate)*up rows"
    route_out = result.region("route_out", torch.float32, (routes, hidden)).cpu()
    rms = float(d["route_out"].pow(2).mean().sqrt())
    assert float((route_out - d["route_out"]).norm() / d["route_out"].norm()) <= 5e-3
    assert float((route_out - d["route_out"]).abs().max()) <= 1e-2 * rms
    merged = oracle.merge_bf16_path(route_out.view(tokens, top_k, hidden), case["topk_weights"])
    assert torch.equal(result.out.cpu().view(torch.int16), merged.view(torch.int16)), "top-k merge order differs"
    _assert_close_bf16(result.out.cpu(), out_ref, "output vs oracle")
