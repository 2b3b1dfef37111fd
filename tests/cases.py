"""Seeded parity cases shared by the golden generator and the tests.

``ref23`` follows the input recipe of the reference's own W8A8 test
(tests/test_moe_w8a8.py:202-211: seed 23, H=I=64, T=48, int8 weights in [-12,12], scales
U(0.0005,0.0035), x ~ 0.3*N(0,1), one expert per token) widened to 2 experts; the others use the
benchmark distributions of fused_cpp_b200.synthetic at small and ragged sizes, and ``cfg1`` is the
benchmark's small W8A8 configuration itself.
"""
from __future__ import annotations

import torch

from fused_cpp_b200 import synthetic
from fused_cpp_b200.synthetic import MoEShape

W8A8_SHAPES = {
    "tiny": MoEShape(tokens=8, hidden=64, inter=64, experts=4, top_k=2),
    "ragged": MoEShape(tokens=37, hidden=144, inter=80, experts=7, top_k=3),
    "wide": MoEShape(tokens=200, hidden=256, inter=128, experts=3, top_k=2),
    "cfg1": synthetic.CONFIG_SMALL_W8A8,
}
W8A8_CASES = ["ref23", "tiny", "ragged", "wide", "cfg1"]
# W8A16 reuses the int8 weights and scales of these W8A8 cases with 16-bit activations (bf16, or their 16-bit fixed-point form).
W8A16_CASES = ["tiny", "ragged", "wide", "cfg1"]

BF16_SHAPES = {
    "tiny": MoEShape(tokens=8, hidden=64, inter=64, experts=4, top_k=2),
    "ragged": MoEShape(tokens=19, hidden=144, inter=80, experts=8, top_k=5),
    "top8": MoEShape(tokens=33, hidden=256, inter=128, experts=16, top_k=8),
    "wide": MoEShape(tokens=300, hidden=128, inter=64, experts=2, top_k=1),
}
BF16_CASES = ["tiny", "ragged", "top8", "wide"]


def _ref23_case() -> dict:
    generator = torch.Generator().manual_seed(23)
    experts, hidden, inter, tokens = 2, 64, 64, 48
    q13 = torch.randint(-12, 13, (experts, 2 * inter, hidden), dtype=torch.int8, generator=generator)
    q2 = torch.randint(-12, 13, (experts, hidden, inter), dtype=torch.int8, generator=generator)
    s13 = torch.rand((experts, 2 * inter), generator=generator) * 0.003 + 0.0005
    s2 = torch.rand((experts, hidden), generator=generator) * 0.003 + 0.0005
    x = (torch.randn((tokens, hidden), generator=generator) * 0.3).to(torch.bfloat16)
    topk_ids = torch.tensor([[token % experts] for token in range(tokens)], dtype=torch.int64)
    topk_weights = torch.ones((tokens, 1), dtype=torch.float32)
    return {"x": x, "w13": q13, "s13": s13, "w2": q2, "s2": s2, "topk_weights": topk_weights, "topk_ids": topk_ids}


def w8a8_case(name: str) -> dict:
    if name == "ref23":
        return _ref23_case()
    shape = W8A8_SHAPES[name]
    case = synthetic.make_w8a8_case(shape, seed=synthetic.SEED_BASE + 1000 * W8A8_CASES.index(name),
                                    skew=(name == "ragged"))
    if name == "ragged":
        # leave one expert without routes and zero one token row (all-zero row quantisation)
        ids = case["topk_ids"]
        case["topk_ids"] = torch.where(ids == 6, torch.full_like(ids, 5), ids)
        case["x"][3].zero_()
    return case


def bf16_case(name: str) -> dict:
    shape = BF16_SHAPES[name]
    std = 0.05 if shape.hidden <= 256 else 0.02
    return synthetic.make_bf16_case(shape, seed=synthetic.SEED_BASE + 5000 + 1000 * BF16_CASES.index(name),
                                    skew=(name == "ragged"), std=std)


# BF16 op variants beyond plain SiLU: (base case, activation of the op, with biases).  For "swigluoai" the case's w13
# (and w13 bias) is in the checkpoint's interleaved layout (row 2j = gate j, row 2j + 1 = up j), as the reference's
# naive implementation reads it (src/fused_cpp/moe/naive.py:39-47).
BF16_VARIANTS = {"bias": ("ragged", "silu", True), "gelu": ("top8", "gelu", False), "gelu_bias": ("tiny", "gelu", True),
                 "swigluoai": ("tiny", "swigluoai", True)}


def bf16_variant_case(name: str) -> dict:
    base, activation, with_bias = BF16_VARIANTS[name]
    case = bf16_case(base)
    case["activation"] = activation
    experts, two_i, hidden = case["w13"].shape
    if with_bias:
        generator = torch.Generator().manual_seed(8800 + sorted(BF16_VARIANTS).index(name))
        case["w13_bias"] = (torch.randn((experts, two_i), generator=generator) * 0.5).to(torch.bfloat16)
        case["w2_bias"] = (torch.randn((experts, hidden), generator=generator) * 0.5).to(torch.bfloat16)
    else:
        case["w13_bias"] = case["w2_bias"] = None
    return case


def gate_then_up(tensor: torch.Tensor) -> torch.Tensor:
    """Interleaved gate/up channels along dim 1 -> gate channels then up channels."""
    count = tensor.shape[1]
    return tensor.index_select(1, torch.cat((torch.arange(0, count, 2), torch.arange(1, count, 2)))).contiguous()


# Dense W8A8 linear cases: (M, K, N, x dtype, out dtype, bias).  The first three are the shapes of the
# reference's own test (tests/test_i8gemm.py:41-47); the others add tile tails and a larger K.
I8GEMM_CASES = {
    "m1": (1, 7, 5, torch.bfloat16, torch.float32, True),
    "m4": (4, 16, 8, torch.bfloat16, torch.bfloat16, True),
    "m9": (9, 31, 13, torch.bfloat16, torch.bfloat16, True),
    "f32": (24, 64, 96, torch.float32, torch.float32, False),
    "wide": (150, 300, 200, torch.bfloat16, torch.bfloat16, False),
    "deep": (40, 2048, 272, torch.bfloat16, torch.float32, True),
    # taller than one 128-row tile: the two-SM kernel's dense epilogue (three 256-row items, two channel blocks, fp32 + bias)
    "tall": (600, 512, 384, torch.bfloat16, torch.float32, True),
    "tall_bf16": (300, 144, 520, torch.bfloat16, torch.bfloat16, False),
    # at most 16 rows, long K, few and ragged channel blocks: the one-SM kernel cuts K into parts that meet in an int32 table
    "skinny": (16, 1536, 200, torch.bfloat16, torch.bfloat16, False),
    "skinny_f32in": (13, 4096, 136, torch.float32, torch.float32, True),
}


# Seed offsets are fixed per name (the committed golden outputs depend on them), not derived from the table's order.
I8GEMM_SEEDS = {"deep": 0, "f32": 1, "m1": 2, "m4": 3, "m9": 4, "wide": 5, "tall": 6, "tall_bf16": 7, "skinny": 8, "skinny_f32in": 9}


def i8gemm_case(name: str) -> dict:
    m, k, n, x_dtype, out_dtype, with_bias = I8GEMM_CASES[name]
    generator = torch.Generator().manual_seed(7000 + I8GEMM_SEEDS[name])
    weight = torch.randint(-16, 17, (n, k), dtype=torch.int8, generator=generator)
    weight_scale = torch.rand(n, generator=generator) * 0.05 + 0.01
    bias = torch.randn(n, generator=generator).to(torch.bfloat16) if with_bias else None
    x = torch.randn((m, k), generator=generator).to(x_dtype)
    if name == "wide":
        x[5].zero_()
    return {"x": x, "weight": weight, "weight_scale": weight_scale, "bias": bias, "out_dtype": out_dtype}
