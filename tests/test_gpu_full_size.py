"""The benchmark's own layer at full size (H = 7168, I = 2048, 256 experts, top-8, T = 8192: `bench.py`'s
`w8a8_prefill_v3_T8192` inputs, 11.5 GB of int8 weights) checked through properties that need no full-size oracle,
plus a chain that ties it to the oracle after all:

  * a token's output depends on nothing but its own row, routes and weights (per-token quantisation, per-route GEMMs,
    per-token merge), so permuting the batch permutes the output bit for bit - although every row then sits in a
    different work item, at a different position of the tile, next to different neighbours;
  * the row tile, and with it the kernel (device-side split of the experts between the one-SM and the two-SM kernel, or
    everything through the two-SM kernel), changes no bit;
  * the fp32 route rows do not depend on the routing weights (those enter in the merge only);
  * the first eight tokens run alone take the decode path (one-SM kernel, 16-row tile) and must give the rows they give
    inside the 8192-token batch; and for those eight tokens the CPU oracle is affordable (64 routes, the experts they hit
    copied to the host), so the full-size prefill result is pinned to the oracle for them, bit for bit.
"""
from __future__ import annotations

import functools

import pytest
import torch

import bench
from fused_cpp_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu

SPEC = bench.WORKLOADS["w8a8_prefill_v3_T8192"]
DIMS = bench.dims_of(SPEC)


@functools.lru_cache(maxsize=None)
def _layer(device_index: int):
    device = torch.device("cuda", device_index)
    return bench.make_experts("int8", device, bench.SEED + 2, range(DIMS["experts"]), DIMS["hidden"], DIMS["inter"])


@functools.lru_cache(maxsize=None)
def _batch():
    return bench.make_batch(SPEC, bench.SEED)


def _forward(device, x, weights, ids, layer, **kw):
    result = _lib.moe_forward(x.to(device), layer["w13"], layer["w2"], weights.to(device), ids.to(device), s13=layer["s13"], s2=layer["s2"], **kw)
    assert result.status()[0] == 0
    return result


def test_full_size_prefill_permutation_tiles_and_routing_weights(cuda_device):
    layer = _layer(cuda_device.index or 0)
    x, weights, ids = _batch()
    tokens, hidden = x.shape
    routes = ids.numel()
    base = _forward(cuda_device, x, weights, ids, layer)
    base_out = base.out.clone()
    base_rows = base.region("route_out", torch.float32, (routes, hidden)).clone()

    permutation = torch.randperm(tokens, generator=torch.Generator().manual_seed(5))
    permuted = _forward(cuda_device, x[permutation], weights[permutation], ids[permutation], layer)
    assert torch.equal(permuted.out.view(torch.int16), base_out[permutation.to(cuda_device)].view(torch.int16)), "output is not permutation-equivariant"
    del permuted

    forced = _forward(cuda_device, x, weights, ids, layer, gate_up_tile=512, down_tile=512)
    assert torch.equal(forced.out.view(torch.int16), base_out.view(torch.int16)), "the row tile changed the output"
    del forced

    rescaled = _forward(cuda_device, x, weights * 2.0, ids, layer)
    rows = rescaled.region("route_out", torch.float32, (routes, hidden))
    assert torch.equal(rows.view(torch.int32), base_rows.view(torch.int32)), "route rows depend on the routing weights"


def test_full_size_prefill_rows_are_pinned_to_the_oracle_through_the_decode_path(cuda_device):
    layer = _layer(cuda_device.index or 0)
    x, weights, ids = _batch()
    hidden = x.shape[1]
    top_k = ids.shape[1]
    few = 8
    big = _forward(cuda_device, x, weights, ids, layer)
    big_out = big.out[:few].cpu()
    big_rows = big.region("route_out", torch.float32, (ids.numel(), hidden))[: few * top_k].cpu()  # rows are in flat route order

    alone = _forward(cuda_device, x[:few], weights[:few], ids[:few], layer)
    assert torch.equal(alone.out.cpu().view(torch.int16), big_out.view(torch.int16)), "decode path and prefill path disagree"
    assert torch.equal(alone.region("route_out", torch.float32, (few * top_k, hidden)).cpu().view(torch.int32), big_rows.view(torch.int32))

    hit = torch.unique(ids[:few])
    remap = torch.full((DIMS["experts"],), -1, dtype=torch.int64)
    remap[hit] = torch.arange(hit.numel())
    on_host = {k: layer[k][hit.to(cuda_device)].cpu() for k in ("w13", "s13", "w2", "s2")}
    expected, dumps = oracle.w8a8_forward(x[:few], on_host["w13"], on_host["s13"], on_host["w2"], on_host["s2"], weights[:few],
                                          remap[ids[:few]], 0, dumps=True)
    assert torch.equal(big_rows.view(torch.int32), dumps["route_out"].view(torch.int32)), "full-size route rows differ from the oracle"
    assert torch.equal(big_out.view(torch.int16), expected.view(torch.int16)), "full-size output differs from the oracle"
