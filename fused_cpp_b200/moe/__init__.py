"""Fused MoE operators: the export list of the reference's `fused_cpp.moe` (src/fused_cpp/moe/__init__.py:67-126)."""
from .bf16_tiled import (  # noqa: F401
    _HAS_BF16_TILED_FUSED_MOE, _HAS_W8A8_TILED_FUSED_MOE, PreparedBF16TiledFusedMoEWeights,
    PreparedBF16TiledRoutedSharedMoEWeights, PreparedW8A8TiledFusedMoEWeights, PreparedW8A8TiledRoutedSharedMoEWeights,
    PreparedW8A16TiledFusedMoEWeights, PreparedW8A16TiledRoutedSharedMoEWeights, available_fused_moe_bf16_tiled_backends,
    bf16_tiled_fused_moe, bf16_tiled_fused_moe_async, bf16_tiled_fused_moe_async_plan, bf16_tiled_fused_moe_planned_staged,
    bf16_tiled_fused_moe_scheduled, bf16_tiled_fused_moe_vllm_staged, fused_moe_bf16_tiled, fused_moe_bf16_tiled_async,
    fused_moe_bf16_tiled_async_plan, fused_moe_bf16_tiled_planned_staged, fused_moe_bf16_tiled_scheduled,
    fused_moe_bf16_tiled_vllm_staged, fused_moe_bf16_tiled_with_shared, fused_moe_tiled, fused_moe_w8a8_tiled,
    fused_moe_w8a8_tiled_async_plan, fused_moe_w8a8_tiled_with_shared, fused_moe_w8a16_tiled,
    fused_moe_w8a16_tiled_async_plan, fused_moe_w8a16_tiled_with_shared, prepare_bf16_tiled_fused_moe_weights,
    prepare_fused_moe_bf16_tiled_weights, prepare_fused_moe_w8a8_tiled_quantized_weights,
    prepare_fused_moe_w8a8_tiled_weights, prepare_fused_moe_w8a16_tiled_quantized_weights,
    prepare_fused_moe_w8a16_tiled_weights, prepare_routed_shared_moe_bf16_tiled_weights,
    prepare_routed_shared_moe_w8a8_tiled_quantized_weights, prepare_routed_shared_moe_w8a16_tiled_quantized_weights,
    prepare_shared_mlp_bf16_tiled_weights, shared_mlp_bf16_tiled)
from .naive import fused_moe_naive, naive_fused_moe  # noqa: F401
from .plan import (  # noqa: F401
    ASYNC_MOE_EXECUTION_STRICT, ASYNC_MOE_EXECUTION_TAIL_POOL, ASYNC_MOE_FULL_EXPERT_RANGE, ASYNC_MOE_PLACEMENT_FIXED,
    ASYNC_MOE_PLACEMENT_TAIL_POOL, ASYNC_MOE_PLAN_VERSION, ASYNC_MOE_RESIZE_NONE, ASYNC_MOE_STAGE_EXPERT, AsyncMoEPlanV2,
    upgrade_legacy_async_plan)
from .planner_runtime import (  # noqa: F401
    DEFAULT_MOE_COST_CACHE_DIR, MoePlannerRuntime, calibrate_moe_planner_quick, enable_moe_planner_quick,
    get_default_moe_planner_runtime, set_default_moe_planner_runtime)

__all__ = [name for name in dir() if not name.startswith("__") and name not in ("bf16_tiled", "naive", "plan", "planner_runtime", "_moe_C")]
