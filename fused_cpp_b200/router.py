"""Router front-end on the GPU: expert scores -> top-k ids and routing weights in the types the MoE ops take.

The reference's operators receive ``topk_weights`` / ``topk_ids`` from their caller
(``src/fused_cpp/moe/naive.py:4-7``); this is the step that produces them, so that a layer can go from router
logits to the MoE output without the ids leaving the GPU:

    weights, ids = router_topk(logits, 8)                        # softmax, top-8, renormalised
    out = fused_cpp_b200.moe.fused_moe_tiled(x, prepared, weights, ids)
"""
from __future__ import annotations

from ._lib import router_topk

__all__ = ["router_topk"]
