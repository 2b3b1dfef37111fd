"""compressed-tensors int8 expert tensors -> the layouts prepare_* take (host logic, no GPU)."""
from __future__ import annotations

import pytest
import torch

from fused_cpp_b200 import checkpoint, synthetic


def _state(experts=3, hidden=32, inter=16, shared=False):
    state, truth = {}, []
    for e in range(experts + (1 if shared else 0)):
        w13, s13, w2, s2 = synthetic.make_int8_expert(hidden, inter, 500 + e)
        if e == 1:  # this expert's gate scales are stored as bf16 in the "checkpoint": the truth is what is stored
            s13 = s13.clone()
            s13[:inter] = s13[:inter].to(torch.bfloat16).float()
        base = f"layers.0.mlp.experts.{e}" if e < experts else "layers.0.mlp.shared_experts"
        state[f"{base}.gate_proj.weight"], state[f"{base}.up_proj.weight"] = w13[:inter].clone(), w13[inter:].clone()
        state[f"{base}.gate_proj.weight_scale"] = s13[:inter].reshape(-1, 1).to(torch.bfloat16 if e == 1 else torch.float32)
        state[f"{base}.up_proj.weight_scale"] = s13[inter:].reshape(-1, 1)
        state[f"{base}.down_proj.weight"], state[f"{base}.down_proj.weight_scale"] = w2.clone(), s2.clone()
        truth.append((w13, s13, w2, s2))
    return state, truth


def test_stacking_matches_the_per_expert_tensors():
    state, truth = _state()
    w13, s13, w2, s2 = checkpoint.stack_compressed_tensors_experts(state, "layers.0.mlp.experts", 3)
    assert w13.shape == (3, 32, 32) and s13.shape == (3, 32) and w2.shape == (3, 32, 16) and s2.shape == (3, 32)
    for e, (tw13, ts13, tw2, ts2) in enumerate(truth):
        assert torch.equal(w13[e], tw13) and torch.equal(w2[e], tw2) and torch.equal(s2[e], ts2)
        assert torch.equal(s13[e], ts13)
    # a callable source and an expert sub-range (expert-parallel shard)
    part = checkpoint.stack_compressed_tensors_experts(lambda name: state[name], "layers.0.mlp.experts", 2, first_expert=1)
    assert torch.equal(part[0][0], truth[1][0]) and torch.equal(part[2][1], truth[2][2])


def test_rejects_what_the_kernels_cannot_take():
    state, _ = _state()
    bad = dict(state)
    bad["layers.0.mlp.experts.0.gate_proj.weight_scale"] = torch.ones(4)  # group-wise scales
    with pytest.raises(ValueError, match="one scale per output channel"):
        checkpoint.stack_compressed_tensors_experts(bad, "layers.0.mlp.experts", 3)
    bad = dict(state)
    bad["layers.0.mlp.experts.2.up_proj.weight"] = bad["layers.0.mlp.experts.2.up_proj.weight"].float()
    with pytest.raises(TypeError, match="torch.int8"):
        checkpoint.stack_compressed_tensors_experts(bad, "layers.0.mlp.experts", 3)
    with pytest.raises(KeyError):
        checkpoint.stack_compressed_tensors_experts(state, "layers.0.mlp.experts", 4)
    with pytest.raises(ValueError, match="mode"):
        checkpoint.prepare_moe_from_compressed_tensors(state, "layers.0.mlp.experts", 3, mode="fp8")


@pytest.mark.gpu
def test_checkpoint_to_forward_w8a16_and_w8a8(cuda_device):
    """The whole route: per-expert checkpoint tensors -> prepared weights (routed + shared) -> forward, against the
    oracle on the stacked tensors."""
    import fused_cpp_b200.moe as moe
    from oracle import oracle
    from tests.test_gpu_bf16 import _assert_close_bf16

    experts, hidden, inter, tokens, top_k = 4, 64, 32, 24, 2
    state, truth = _state(experts, hidden, inter, shared=True)
    topk_w, topk_ids = synthetic.make_routing(tokens, experts, top_k, 77)
    x = synthetic.make_activations(tokens, hidden, 78)
    all_ids = torch.cat((topk_ids, torch.full((tokens, 1), experts, dtype=torch.int64)), 1)
    all_w = torch.cat((topk_w, torch.ones((tokens, 1))), 1)
    stacked = [torch.stack([t[i] for t in truth]) for i in range(4)]
    previous = moe.set_default_moe_planner_runtime(moe.MoePlannerRuntime(None, hidden_size=hidden, intermediate_size=inter, global_experts=experts,
                                                                          local_experts=experts, shared_experts=1))
    try:
        for mode, op, reference in (("w8a16", moe.fused_moe_w8a16_tiled_with_shared, oracle.w8a16_forward),
                                    ("w8a8", moe.fused_moe_w8a8_tiled_with_shared, oracle.w8a8_forward)):
            prepared = checkpoint.prepare_moe_from_compressed_tensors(state, "layers.0.mlp.experts", experts, mode=mode,
                                                                      shared_prefix="layers.0.mlp.shared_experts")
            assert prepared.shared_expert_id == experts and prepared.packed.w13[0].shape[0] == experts + 1
            out = op(x.to(cuda_device), prepared, topk_w.to(cuda_device), topk_ids.to(cuda_device))
            expected = reference(x, stacked[0], stacked[1], stacked[2], stacked[3], all_w, all_ids)
            if mode == "w8a8":
                assert torch.equal(out.cpu().view(torch.int16), expected.view(torch.int16))
            else:
                _assert_close_bf16(out.cpu(), expected, "W8A16 from a checkpoint")
    finally:
        moe.set_default_moe_planner_runtime(previous)
