"""A bounded peer-barrier wait that runs out, on one GPU, with nothing left waiting and no fault.

Two expert-parallel contexts ("rank 0" and "rank 1") are created in this process on the same GPU and
connected by slab address.  Rank 0 runs a whole forward while rank 1 does nothing: every barrier of rank 0
waits for a flag that nobody sets, gives up after the 50 ms limit and records FMOE_ERR_DEVICE_WAIT with the
rank it waited for.  The rest of that forward must then send nothing and multiply nothing: no row, scale or
return address is stored in either slab.  Rank 1 runs its three calls afterwards (late): its waits are
satisfied at once by the flags rank 0 already raised, and it finishes without an error.  The kernels of the
two ranks never run at the same time (one stream, one after the other), so nothing here spins on a kernel
that is not resident.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from fused_cpp_b200 import _lib
from tests import cases

pytestmark = pytest.mark.gpu

WORLD, TOKENS, TOP_K, HIDDEN, INTER, LOCAL_EXPERTS = 2, 8, 2, 64, 64, 2


def _read_device(address: int, nbytes: int) -> torch.Tensor:
    from cuda.bindings import runtime

    host = torch.empty(nbytes, dtype=torch.uint8)
    (error,) = runtime.cudaMemcpy(host.data_ptr(), address, nbytes, runtime.cudaMemcpyKind.cudaMemcpyDeviceToHost)
    assert int(error) == 0, error
    return host


def _forward(context, case, device, weights):
    config = _lib.Config()
    config.swiglu_limit = 10.0
    x = case["x"].to(device)
    ids = case["topk_ids"].to(device)
    out = torch.zeros((TOKENS, HIDDEN), dtype=torch.bfloat16, device=device)
    context.dispatch(x, ids, WORLD * LOCAL_EXPERTS, -1, 0)
    context.experts(weights["w13"], weights["s13"], weights["w2"], weights["s2"], config)
    context.combine(case["topk_weights"].to(device), TOKENS, False, out)
    return out


def test_peer_barrier_wait_runs_out_and_the_forward_stores_nothing(cuda_device, monkeypatch):
    monkeypatch.setenv("FUSED_CPP_MOE_EP_WAIT_MS", "50")
    case = cases.w8a8_case("tiny")  # 8 tokens, H = I = 64, 4 experts, top-2
    assert case["x"].shape == (TOKENS, HIDDEN) and case["w13"].shape[0] == WORLD * LOCAL_EXPERTS
    contexts = [_lib.PeerContext(WORLD, rank, TOKENS, TOP_K, HIDDEN, INTER, LOCAL_EXPERTS, True) for rank in range(WORLD)]
    try:
        addresses = [context.slab_address for context in contexts]
        for context in contexts:
            context.connect_addresses(addresses)
        weights = [{k: case[k][rank * LOCAL_EXPERTS:(rank + 1) * LOCAL_EXPERTS].to(cuda_device).contiguous()
                    for k in ("w13", "s13", "w2", "s2")} for rank in range(WORLD)]

        _forward(contexts[0], case, cuda_device, weights[0])
        dispatch_error, expert_error = contexts[0].read_status()
        text = _lib.load().fmoe_last_error().decode()
        assert dispatch_error == _lib.ERR_DEVICE_WAIT and expert_error == _lib.ERR_DEVICE_WAIT
        assert "waiting for rank 1" in text, text

        # Slab layout: rows, scales, return addresses and result rows first, then the count table (one row of
        # world * local_experts + 1 ints per rank) and the barrier flags, each region padded to 256 bytes.  Only the
        # table and the flags may have been written (rank 0 publishes its counts and its epochs before it waits).
        tail = 256 + 256
        for context in contexts:
            body = _read_device(context.slab_address, context.slab_bytes - tail)
            assert int(body.count_nonzero()) == 0, "a row, scale, return address or result row was stored after the failed barrier"

        # The late rank: every flag it waits for is already there.
        _forward(contexts[1], case, cuda_device, weights[1])
        dispatch_error, expert_error = contexts[1].read_status()
        assert (dispatch_error, expert_error) == (0, 0)
        torch.cuda.synchronize()
    finally:
        torch.cuda.synchronize()
        for context in contexts:
            context.close()
