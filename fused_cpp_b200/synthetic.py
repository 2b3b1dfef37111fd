"""Seeded synthetic inputs for the routed-expert MoE layer.

The benchmark configurations name no dataset: router logits, activations and weights are drawn
from fixed distributions.  Everything is generated with a CPU ``torch.Generator`` so that the
CUDA path and a CPU checker see identical bits; the large weight sets of the DeepSeek-V3-scale
layer are generated per expert (seed = base + expert) so that a checker can rebuild only the
experts a routing actually hits.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

SEED_BASE = 20260101


@dataclass(frozen=True)
class MoEShape:
    tokens: int
    hidden: int
    inter: int
    experts: int
    top_k: int


CONFIG_SMALL_W8A8 = MoEShape(tokens=16, hidden=2048, inter=1024, experts=16, top_k=4)
CONFIG_V3 = MoEShape(tokens=64, hidden=7168, inter=2048, experts=256, top_k=8)


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


def zipf_bias(experts: int, seed: int) -> torch.Tensor:
    """bias_e = 2*ln(1/(rank_e+1)) over a seeded random ranking of the experts."""
    rank = torch.randperm(experts, generator=_gen(seed)).to(torch.float32)
    return 2.0 * torch.log(1.0 / (rank + 1.0))


def make_routing(tokens: int, experts: int, top_k: int, seed: int = SEED_BASE, skew: bool = False):
    """Router logits N(0,1) [+ Zipf bias] -> softmax -> top-k -> weights renormalised to sum 1.

    Returns (topk_weights fp32 [T,K], topk_ids int64 [T,K]).
    """
    logits = torch.randn((tokens, experts), generator=_gen(seed), dtype=torch.float32)
    if skew:
        logits = logits + zipf_bias(experts, seed + 100)
    probs = torch.softmax(logits, dim=-1)
    weights, ids = torch.topk(probs, top_k, dim=-1)
    weights = weights / weights.sum(dim=-1, keepdim=True)
    return weights.contiguous(), ids.to(torch.int64).contiguous()


def make_activations(tokens: int, hidden: int, seed: int = SEED_BASE + 1) -> torch.Tensor:
    return torch.randn((tokens, hidden), generator=_gen(seed), dtype=torch.float32).to(torch.bfloat16)


def make_int8_expert(hidden: int, inter: int, seed: int):
    """One expert's W8A8 weights: int8 uniform in [-127,127], per-output-channel fp32 scales
    U(0.5,2)/(127*sqrt(K_in)).  Returns (w13[2I,H], s13[2I], w2[H,I], s2[H])."""
    g = _gen(seed)
    w13 = torch.randint(-127, 128, (2 * inter, hidden), generator=g, dtype=torch.int8)
    w2 = torch.randint(-127, 128, (hidden, inter), generator=g, dtype=torch.int8)
    s13 = (torch.rand(2 * inter, generator=g) * 1.5 + 0.5) / (127.0 * math.sqrt(hidden))
    s2 = (torch.rand(hidden, generator=g) * 1.5 + 0.5) / (127.0 * math.sqrt(inter))
    return w13, s13.to(torch.float32), w2, s2.to(torch.float32)


def make_bf16_expert(hidden: int, inter: int, seed: int, std: float = 0.02):
    """One expert's BF16 weights N(0, std^2): (w13[2I,H], w2[H,I])."""
    g = _gen(seed)
    w13 = (torch.randn((2 * inter, hidden), generator=g) * std).to(torch.bfloat16)
    w2 = (torch.randn((hidden, inter), generator=g) * std).to(torch.bfloat16)
    return w13, w2


def make_int8_weights(shape: MoEShape, seed: int = SEED_BASE + 2):
    """All experts stacked: (w13[E,2I,H] i8, s13[E,2I], w2[E,H,I] i8, s2[E,H])."""
    parts = [make_int8_expert(shape.hidden, shape.inter, seed + e) for e in range(shape.experts)]
    return tuple(torch.stack([p[i] for p in parts]).contiguous() for i in range(4))


def make_bf16_weights(shape: MoEShape, seed: int = SEED_BASE + 2, std: float = 0.02):
    parts = [make_bf16_expert(shape.hidden, shape.inter, seed + e, std) for e in range(shape.experts)]
    return tuple(torch.stack([p[i] for p in parts]).contiguous() for i in range(2))


def make_w8a8_case(shape: MoEShape, seed: int = SEED_BASE, skew: bool = False) -> dict:
    topk_w, topk_ids = make_routing(shape.tokens, shape.experts, shape.top_k, seed, skew)
    w13, s13, w2, s2 = make_int8_weights(shape, seed + 2)
    return {"x": make_activations(shape.tokens, shape.hidden, seed + 1), "w13": w13, "s13": s13, "w2": w2, "s2": s2,
            "topk_weights": topk_w, "topk_ids": topk_ids}


def make_bf16_case(shape: MoEShape, seed: int = SEED_BASE, skew: bool = False, std: float = 0.02) -> dict:
    topk_w, topk_ids = make_routing(shape.tokens, shape.experts, shape.top_k, seed, skew)
    w13, w2 = make_bf16_weights(shape, seed + 2, std)
    return {"x": make_activations(shape.tokens, shape.hidden, seed + 1), "w13": w13, "w2": w2,
            "topk_weights": topk_w, "topk_ids": topk_ids}


def algorithmic_work(shape: MoEShape, topk_ids: torch.Tensor, weight_bytes: int, shared: bool = False) -> dict:
    """Algorithmic bytes and operations of one layer call.

    bytes = weights of the experts this routing actually hits (+ per-channel scales for int8)
            + x in + out + top-k arrays;   ops = 2 * routes * 3 * H * I.
    """
    active = int(torch.unique(topk_ids).numel()) + (1 if shared else 0)
    h, i = shape.hidden, shape.inter
    per_expert = 3 * h * i * weight_bytes + ((2 * i + h) * 4 if weight_bytes == 1 else 0)
    tokens = topk_ids.shape[0]
    k = topk_ids.shape[1]
    act = tokens * h * 2 * 2 + tokens * k * (4 + 8)
    routes = tokens * k + (tokens if shared else 0)
    return {"active_experts": active, "bytes": active * per_expert + act, "ops": 2 * routes * 3 * h * i}
