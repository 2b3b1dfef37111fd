"""Plain-PyTorch routed-expert FFN, the readable reference of the op's tensor semantics
(the role of src/fused_cpp/moe/naive.py in the reference; device-agnostic).

topk_weights / topk_ids come from the router; tokens are grouped by expert (stable order), each
expert runs gate_up -> activation -> down, and the K expert outputs of a token are weighted and summed.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.nn.functional as F

__all__ = ["fused_moe_naive", "naive_fused_moe"]


def _activation(name: Any):
    name = getattr(name, "value", name)
    if name == "silu":
        return lambda x: F.silu(x[..., : x.shape[-1] // 2]) * x[..., x.shape[-1] // 2:]
    if name == "gelu":
        return lambda x: F.gelu(x[..., : x.shape[-1] // 2]) * x[..., x.shape[-1] // 2:]
    if name == "swigluoai":
        def swigluoai(x, alpha=1.702, limit=7.0):
            gate, up = x[..., ::2].clamp(max=limit), x[..., 1::2].clamp(-limit, limit)
            return (up + 1) * gate * torch.sigmoid(gate * alpha)
        return swigluoai
    raise ValueError(f"Unsupported MoE activation {name!r}; supported activations: gelu, silu, swigluoai")


def fused_moe_naive(input, w13_weight, w2_weight, topk_weights, topk_ids, *, w13_bias=None, w2_bias=None,
                    activation: Any = "silu", global_num_experts: int = -1, skip_weighted: bool = False, out=None):
    act = _activation(activation)
    if input.dim() != 2 or w13_weight.dim() != 3 or w2_weight.dim() != 3:
        raise ValueError("input must be [T, H]; w13 [E, 2F, H]; w2 [E, H, F]")
    if topk_ids.shape != topk_weights.shape or topk_ids.dim() != 2 or topk_ids.shape[0] != input.shape[0]:
        raise ValueError("topk_ids and topk_weights must both be [T, K]")
    experts = w13_weight.shape[0] if global_num_experts < 0 else int(global_num_experts)
    if experts > w13_weight.shape[0]:
        raise ValueError("global_num_experts cannot exceed available expert weights")
    tokens, hidden = input.shape
    top_k = topk_ids.shape[1]
    if skip_weighted and top_k != 1:
        raise AssertionError("skip_weighted is only valid when top_k == 1")
    if topk_ids.numel() and (int(topk_ids.min()) < 0 or int(topk_ids.max()) >= experts):
        raise ValueError("topk_ids out of range")
    flat = topk_ids.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    rows = input.index_select(0, order // top_k)
    counts = torch.bincount(flat, minlength=experts).tolist()
    pieces, begin = [], 0
    for expert, count in enumerate(counts):
        if count == 0:
            continue
        block = rows[begin:begin + count]
        mid = act(F.linear(block, w13_weight[expert], None if w13_bias is None else w13_bias[expert]))
        pieces.append(F.linear(mid, w2_weight[expert], None if w2_bias is None else w2_bias[expert]))
        begin += count
    sorted_out = torch.cat(pieces, 0) if pieces else input.new_empty((0, hidden))
    per_route = torch.empty_like(sorted_out)
    per_route[order] = sorted_out
    if skip_weighted:
        result = per_route
    else:
        result = (per_route.view(tokens, top_k, hidden).to(topk_weights.dtype) * topk_weights.unsqueeze(-1)).sum(1).to(per_route.dtype)
    if out is not None:
        out.copy_(result)
        return out
    return result


naive_fused_moe = fused_moe_naive
