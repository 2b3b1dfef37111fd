"""Public fused-MoE wrappers with the reference's signatures (src/fused_cpp/moe/bf16_tiled.py).

Prepared-weight holders, `prepare_*`, the BF16 and W8A8 forwards, the type-dispatching
`fused_moe_tiled`, the routed+shared wrappers and the standalone shared MLP.  The one deliberate
change of contract: forward ops take CUDA tensors and `prepare_*` return CUDA-resident weights
(the reference is CPU-only).  Nothing here reads `topk_ids` on the host: range checks happen in
the route-build kernel and surface through the status block.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Tuple

import torch

from . import _moe_C as _native
from .plan import AsyncMoEPlanV2, gpu_placeholder_plan

PreparedWeight = Tuple[torch.Tensor, int, int]
_INTEGER_DTYPES = {torch.int8, torch.int16, torch.int32, torch.int64}


@dataclass(frozen=True)
class PreparedBF16TiledFusedMoEWeights:
    """BF16 expert weights resident on the GPU: w13 = (tensor[E,2F,H], K=H, N=2F), w2 = (tensor[E,H,F], K=F, N=H)."""
    w13: PreparedWeight
    w2: PreparedWeight
    fused_silu: bool = False
    gemm_backend: int = _native.BACKEND_ID
    backend_n_tile: int = _native.BACKEND_N_TILE
    backend_name: str = _native.BACKEND_NAME


@dataclass(frozen=True)
class PreparedW8A16TiledFusedMoEWeights:
    """Per-output-channel int8 expert weights + fp32 scales for the W8A16 path (16-bit activations: 16-bit fixed point per
    row by default, or bf16 as they are with FUSED_CPP_MOE_W8A16_FORM=bf16)."""
    w13: tuple[torch.Tensor, int, int, torch.Tensor]
    w2: tuple[torch.Tensor, int, int, torch.Tensor]
    fused_silu: bool = True
    gemm_backend: int = _native.BACKEND_ID
    backend_n_tile: int = _native.BACKEND_N_TILE
    backend_name: str = _native.W8A16_BACKEND_NAME


@dataclass(frozen=True)
class PreparedW8A8TiledFusedMoEWeights:
    """Per-output-channel int8 expert weights + fp32 scales for the dynamic-activation W8A8 path."""
    w13: tuple[torch.Tensor, int, int, torch.Tensor]
    w2: tuple[torch.Tensor, int, int, torch.Tensor]
    fused_silu: bool = True
    gemm_backend: int = _native.BACKEND_ID
    backend_n_tile: int = _native.BACKEND_N_TILE
    backend_name: str = _native.W8A8_BACKEND_NAME


@dataclass(frozen=True)
class PreparedBF16TiledRoutedSharedMoEWeights:
    packed: PreparedBF16TiledFusedMoEWeights
    routed_experts: int
    shared_expert_id: int


@dataclass(frozen=True)
class PreparedW8A16TiledRoutedSharedMoEWeights:
    packed: PreparedW8A16TiledFusedMoEWeights
    routed_experts: int
    shared_expert_id: int


@dataclass(frozen=True)
class PreparedW8A8TiledRoutedSharedMoEWeights:
    packed: PreparedW8A8TiledFusedMoEWeights
    routed_experts: int
    shared_expert_id: int


_HAS_BF16_TILED_FUSED_MOE = bool(_native.fused_moe_bf16_tiled_available_backends())
_HAS_W8A8_TILED_FUSED_MOE = bool(_native.fused_moe_w8a8_tiled_available())

# The native ops the wrappers call, under the module-level names the reference binds them to
# (src/fused_cpp/moe/bf16_tiled.py:87-96), so that callers and tests that substitute an op find the same hook.
# The wrappers below validate types and shapes only; the rule that tensors live on a CUDA device belongs to the
# native ops.
_fused_moe_bf16_tiled_impl = _native.fused_moe_bf16_tiled
_fused_moe_bf16_tiled_async_plan_v2_impl = _native.fused_moe_bf16_tiled_async_plan_v2
_fused_moe_w8a8_async_plan_v2_impl = _native.fused_moe_w8a8_tiled_async_plan_v2
_shared_mlp_bf16_tiled_impl = _native.shared_mlp_bf16_tiled
_fused_moe_w8a16_async_plan_v2_impl = _native.fused_moe_w8a16_tiled_async_plan_v2


def _require_backend() -> None:
    if not _HAS_BF16_TILED_FUSED_MOE:
        raise RuntimeError("the B200 fused MoE backend is unavailable: no compute-capability-10.x CUDA device "
                           "(there is no CPU fallback)")


def available_fused_moe_bf16_tiled_backends() -> tuple[str, ...]:
    return tuple(_native.fused_moe_bf16_tiled_available_backends())


def _activation_name(activation: Any) -> str:
    value = getattr(activation, "value", activation)
    return value if isinstance(value, str) else str(value)


def _native_activation_name(activation: Any, weights: Any, swiglu_limit: float | None) -> str:
    """Activation string of the native op (bf16_tiled.py:245-260).  Every prepared weight of this backend supports
    the clamp-10 variant, so `weights` takes no part in the decision."""
    name = _activation_name(activation)
    if swiglu_limit is None or float(swiglu_limit) == 0.0:
        return name
    if not math.isfinite(float(swiglu_limit)) or float(swiglu_limit) != 10.0:
        raise ValueError("clamped SwiGLU currently requires swiglu_limit=10.0")
    if name != "silu":
        raise ValueError("swiglu_limit is only valid with activation='silu'")
    return "silu_clamp10"


def _validate_output_buffer(input: torch.Tensor, out: torch.Tensor | None) -> None:
    if out is None:
        return
    if not isinstance(out, torch.Tensor):
        raise TypeError("out must be a torch.Tensor or None")
    if out.dtype != torch.bfloat16 or out.device != input.device:
        raise ValueError("out must be a BF16 tensor on the input's device")
    if tuple(out.shape) != tuple(input.shape) or not out.is_contiguous():
        raise ValueError("out must be contiguous and match the input shape")


def _check_forward_inputs(input, topk_weights, topk_ids, num_threads) -> None:
    if input.dtype != torch.bfloat16:
        raise TypeError(f"input must be torch.bfloat16, got {input.dtype}")
    if topk_ids.dtype not in _INTEGER_DTYPES:
        raise TypeError(f"topk_ids must use an integer dtype, got {topk_ids.dtype}")
    if not topk_weights.dtype.is_floating_point:
        raise TypeError(f"topk_weights must use a floating dtype, got {topk_weights.dtype}")
    if int(num_threads) <= 0:
        raise ValueError(f"num_threads must be positive, got {num_threads}")


# ---- prepare -------------------------------------------------------------------------------------

def prepare_fused_moe_bf16_tiled_weights(w13_weight, w2_weight, *, fuse_silu: bool = False, backend: str = "auto"):
    """w13 [E,2F,H], w2 [E,H,F] bf16 (CPU or CUDA) -> GPU-resident prepared weights (bf16_tiled.py:396)."""
    _require_backend()
    if w13_weight.dtype != torch.bfloat16 or w2_weight.dtype != torch.bfloat16:
        raise TypeError("BF16 tiled fused MoE weights must be torch.bfloat16")
    if not isinstance(backend, str):
        raise TypeError(f"backend must be a string, got {type(backend).__name__}")
    packed = _native.fused_moe_bf16_tiled_prepare_weights(w13_weight, w2_weight, bool(fuse_silu), backend)
    return PreparedBF16TiledFusedMoEWeights(w13=(packed[0], int(packed[1]), int(packed[2])), w2=(packed[3], int(packed[4]), int(packed[5])),
                                            fused_silu=bool(fuse_silu), gemm_backend=int(packed[6]), backend_n_tile=int(packed[7]),
                                            backend_name=str(packed[8]))


prepare_bf16_tiled_fused_moe_weights = prepare_fused_moe_bf16_tiled_weights


def prepare_shared_mlp_bf16_tiled_weights(w13_weight, w2_weight, *, backend: str = "auto"):
    """One shared expert [2F,H] / [H,F] as a single-expert prepared object."""
    if w13_weight.dim() != 2 or w2_weight.dim() != 2:
        raise ValueError("shared MLP weights must be [2F, H] and [H, F]")
    return prepare_fused_moe_bf16_tiled_weights(w13_weight.unsqueeze(0), w2_weight.unsqueeze(0), fuse_silu=True, backend=backend)


def prepare_routed_shared_moe_bf16_tiled_weights(routed_w13_weight, routed_w2_weight, shared_w13_weight, shared_w2_weight, *,
                                                 backend: str = "auto"):
    _require_backend()
    packed = _native.fused_moe_bf16_tiled_prepare_routed_shared_weights(routed_w13_weight, routed_w2_weight, shared_w13_weight,
                                                                        shared_w2_weight, backend)
    routed = int(routed_w13_weight.shape[0])
    holder = PreparedBF16TiledFusedMoEWeights(w13=(packed[0], int(packed[1]), int(packed[2])), w2=(packed[3], int(packed[4]), int(packed[5])),
                                              fused_silu=True, gemm_backend=int(packed[6]), backend_n_tile=int(packed[7]),
                                              backend_name=str(packed[8]))
    return PreparedBF16TiledRoutedSharedMoEWeights(packed=holder, routed_experts=routed, shared_expert_id=routed)


def _prepared_w8a8(packed) -> PreparedW8A8TiledFusedMoEWeights:
    return PreparedW8A8TiledFusedMoEWeights(w13=(packed[0], int(packed[1]), int(packed[2]), packed[3]),
                                            w2=(packed[4], int(packed[5]), int(packed[6]), packed[7]),
                                            gemm_backend=int(packed[8]), backend_n_tile=int(packed[9]))


def prepare_fused_moe_w8a8_tiled_weights(w13_weight, w2_weight):
    """Quantise bf16 expert weights per output channel (on the GPU) for dynamic W8A8 (bf16_tiled.py:511)."""
    _require_backend()
    if w13_weight.dtype != torch.bfloat16 or w2_weight.dtype != torch.bfloat16:
        raise TypeError("W8A8 source weights must be torch.bfloat16")
    return _prepared_w8a8(_native.fused_moe_w8a8_tiled_prepare_weights(w13_weight, w2_weight))


def prepare_fused_moe_w8a8_tiled_quantized_weights(w13_weight, w13_scale, w2_weight, w2_scale):
    """Checkpoint int8 weights + per-output-channel scales -> prepared W8A8 weights (bf16_tiled.py:526)."""
    _require_backend()
    return _prepared_w8a8(_native.fused_moe_w8a8_tiled_prepare_quantized_weights(w13_weight, w13_scale, w2_weight, w2_scale))


def prepare_routed_shared_moe_w8a8_tiled_quantized_weights(routed_w13_weight, routed_w13_scale, routed_w2_weight, routed_w2_scale,
                                                           shared_w13_weight, shared_w13_scale, shared_w2_weight, shared_w2_scale):
    """Routed experts followed by the shared expert as expert id E (bf16_tiled.py:575-612)."""
    if shared_w13_weight.dim() != 2 or shared_w2_weight.dim() != 2:
        raise ValueError("shared W8A8 weights must be [2F, H] and [H, F]")
    experts = routed_w13_weight.shape[0]
    packed = prepare_fused_moe_w8a8_tiled_quantized_weights(
        torch.cat((routed_w13_weight, shared_w13_weight.unsqueeze(0)), dim=0),
        torch.cat((routed_w13_scale.reshape(experts, -1), shared_w13_scale.reshape(1, -1)), dim=0),
        torch.cat((routed_w2_weight, shared_w2_weight.unsqueeze(0)), dim=0),
        torch.cat((routed_w2_scale.reshape(experts, -1), shared_w2_scale.reshape(1, -1)), dim=0))
    return PreparedW8A8TiledRoutedSharedMoEWeights(packed=packed, routed_experts=int(experts), shared_expert_id=int(experts))


def _prepared_w8a16(packed) -> PreparedW8A16TiledFusedMoEWeights:
    return PreparedW8A16TiledFusedMoEWeights(w13=(packed[0], int(packed[1]), int(packed[2]), packed[3]),
                                             w2=(packed[4], int(packed[5]), int(packed[6]), packed[7]),
                                             gemm_backend=int(packed[8]), backend_n_tile=int(packed[9]))


def prepare_fused_moe_w8a16_tiled_weights(w13_weight, w2_weight):
    """Quantise bf16 expert weights to symmetric per-output-channel int8 on the GPU (bf16_tiled.py:453)."""
    _require_backend()
    if w13_weight.dtype != torch.bfloat16 or w2_weight.dtype != torch.bfloat16:
        raise TypeError("W8A16 source weights must be torch.bfloat16")
    return _prepared_w8a16(_native.fused_moe_w8a16_tiled_prepare_weights(w13_weight, w2_weight))


def prepare_fused_moe_w8a16_tiled_quantized_weights(w13_weight, w13_scale, w2_weight, w2_scale):
    """Checkpoint int8 weights + per-output-channel scales (compressed-tensors style) -> prepared W8A16 weights
    (bf16_tiled.py:483; docs/vllm_bf16_tiled_moe_integration.md:252-259)."""
    _require_backend()
    if w13_weight.dtype != torch.int8 or w2_weight.dtype != torch.int8:
        raise TypeError("W8A16 quantized weights must be torch.int8")
    return _prepared_w8a16(_native.fused_moe_w8a16_tiled_prepare_quantized_weights(w13_weight, w13_scale.to(torch.float32),
                                                                                   w2_weight, w2_scale.to(torch.float32)))


def prepare_routed_shared_moe_w8a16_tiled_quantized_weights(routed_w13_weight, routed_w13_scale, routed_w2_weight, routed_w2_scale,
                                                            shared_w13_weight, shared_w13_scale, shared_w2_weight, shared_w2_scale):
    """Routed experts followed by the shared expert as expert id E (bf16_tiled.py:541)."""
    _require_backend()
    packed = _native.fused_moe_w8a16_tiled_prepare_quantized_routed_shared_weights(
        routed_w13_weight, routed_w13_scale.to(torch.float32), routed_w2_weight, routed_w2_scale.to(torch.float32),
        shared_w13_weight, shared_w13_scale.to(torch.float32), shared_w2_weight, shared_w2_scale.to(torch.float32))
    experts = int(routed_w13_weight.shape[0])
    return PreparedW8A16TiledRoutedSharedMoEWeights(packed=_prepared_w8a16(packed), routed_experts=experts, shared_expert_id=experts)


# ---- forward -------------------------------------------------------------------------------------

def _plan_args(plan: AsyncMoEPlanV2):
    """The plan as the native op's positional arguments.  Plans are frozen, so the tuple is built once per plan object
    and kept on it."""
    cached = plan.__dict__.get("_native_args")
    if cached is None:
        cached = _build_plan_args(plan)
        object.__setattr__(plan, "_native_args", cached)
    return cached


def _build_plan_args(plan: AsyncMoEPlanV2):
    def i64(t):
        return t.to(torch.int64).contiguous()
    return (i64(plan.task_expert_ids), i64(plan.task_core_begins), i64(plan.task_threads), i64(plan.task_dep_offsets),
            i64(plan.task_deps), plan.plan_version, plan.native_execution_mode, i64(plan.task_preferred_threads),
            i64(plan.task_min_threads), i64(plan.task_max_threads), i64(plan.task_allowed_thread_offsets),
            i64(plan.task_allowed_threads), i64(plan.task_placement_modes), i64(plan.task_numa_nodes), i64(plan.task_stage_ids),
            i64(plan.task_resize_points), i64(plan.task_range_granularities), i64(plan.task_w13_window_tiles),
            i64(plan.task_w2_window_tiles), i64(plan.thread_cpu_ids))


def fused_moe_bf16_tiled_async_plan(input, weights, topk_weights, topk_ids, plan, *, w13_bias=None, w2_bias=None,
                                    activation: Any = "silu", global_num_experts: int = -1, skip_weighted: bool = False,
                                    silu_poly_degree: int = 5, swiglu_limit: float | None = None, out=None):
    """BF16 forward under an explicit Plan V2 (bf16_tiled.py:1224)."""
    if _fused_moe_bf16_tiled_async_plan_v2_impl is None:
        raise RuntimeError("BF16 tiled fused MoE Plan V2 requires native fused_moe_bf16_tiled_async_plan_v2 support")
    if not all(hasattr(weights, name) for name in ("w13", "w2", "fused_silu", "gemm_backend", "backend_n_tile")):
        raise TypeError("weights must be PreparedBF16TiledFusedMoEWeights")
    _check_forward_inputs(input, topk_weights, topk_ids, 1)
    _validate_output_buffer(input, out)
    materialized = plan if isinstance(plan, AsyncMoEPlanV2) else AsyncMoEPlanV2.from_dict(plan)
    result = _fused_moe_bf16_tiled_async_plan_v2_impl(
        input.contiguous(), weights.w13[0], weights.w13[1], weights.w13[2], weights.w2[0], weights.w2[1], weights.w2[2],
        topk_weights.to(torch.float32).contiguous(), topk_ids.to(torch.int64).contiguous(), *_plan_args(materialized),
        w13_bias, w2_bias, materialized.num_threads, _native_activation_name(activation, weights, swiglu_limit), int(global_num_experts),
        bool(skip_weighted), bool(weights.fused_silu), int(silu_poly_degree), int(weights.gemm_backend),
        int(weights.backend_n_tile), out, materialized.native_early_merge)
    return out if out is not None else result


def fused_moe_bf16_tiled(input, weights, topk_weights, topk_ids, *, w13_bias=None, w2_bias=None, num_threads: int = 1,
                         activation: Any = "silu", global_num_experts: int = -1, skip_weighted: bool = False,
                         silu_poly_degree: int = 5, swiglu_limit: float | None = None, out=None):
    """BF16 routed-expert forward (bf16_tiled.py:676).  With an installed planner runtime the call goes
    through Plan V2 (which carries the calibrated row tiles); otherwise the op picks its tiles itself."""
    _require_backend()
    if not isinstance(weights, PreparedBF16TiledFusedMoEWeights):
        raise TypeError("weights must be PreparedBF16TiledFusedMoEWeights")
    _check_forward_inputs(input, topk_weights, topk_ids, num_threads)
    _validate_output_buffer(input, out)
    from .planner_runtime import get_default_moe_planner_runtime

    runtime = get_default_moe_planner_runtime()
    if runtime is not None:
        plan = runtime.plan_for_dispatch(weights, topk_ids, num_threads=int(num_threads), activation=activation,
                                         global_num_experts=int(global_num_experts))
        if plan is not None:
            return fused_moe_bf16_tiled_async_plan(input, weights, topk_weights, topk_ids, plan, w13_bias=w13_bias, w2_bias=w2_bias,
                                                   activation=activation, global_num_experts=global_num_experts,
                                                   skip_weighted=skip_weighted, silu_poly_degree=silu_poly_degree,
                                                   swiglu_limit=swiglu_limit, out=out)
    result = _fused_moe_bf16_tiled_impl(
        input.contiguous(), weights.w13[0], weights.w13[1], weights.w13[2], weights.w2[0], weights.w2[1], weights.w2[2],
        topk_weights.to(torch.float32).contiguous(), topk_ids.to(torch.int64).contiguous(), w13_bias, w2_bias, int(num_threads),
        _native_activation_name(activation, weights, swiglu_limit), int(global_num_experts), bool(skip_weighted), bool(weights.fused_silu),
        int(silu_poly_degree), int(weights.gemm_backend), int(weights.backend_n_tile), out)
    return out if out is not None else result


bf16_tiled_fused_moe = fused_moe_bf16_tiled
bf16_tiled_fused_moe_async_plan = fused_moe_bf16_tiled_async_plan


def fused_moe_bf16_tiled_scheduled(input, weights, topk_weights, topk_ids, wave_offsets, team_expert_ids, team_threads, *,
                                   thread_cpu_ids=None, **kwargs):
    """Wave-scheduled variant: the schedule describes CPU teams and is ignored on the GPU."""
    kwargs.pop("num_threads", None)
    return fused_moe_bf16_tiled(input, weights, topk_weights, topk_ids, **kwargs)


def fused_moe_bf16_tiled_async(input, weights, topk_weights, topk_ids, task_expert_ids, task_core_begins, task_threads,
                               task_dep_offsets, task_deps, *, thread_cpu_ids=None, **kwargs):
    """Async-DAG variant: the task graph describes CPU teams and is ignored on the GPU."""
    kwargs.pop("num_threads", None)
    return fused_moe_bf16_tiled(input, weights, topk_weights, topk_ids, **kwargs)


bf16_tiled_fused_moe_scheduled = fused_moe_bf16_tiled_scheduled
bf16_tiled_fused_moe_async = fused_moe_bf16_tiled_async


def fused_moe_bf16_tiled_planned_staged(*_args, **_kwargs):
    raise RuntimeError("fused_moe_bf16_tiled_planned_staged is not implemented on this backend "
                       "(a CPU scheduling comparison path)")


def fused_moe_bf16_tiled_vllm_staged(*_args, **_kwargs):
    raise RuntimeError("fused_moe_bf16_tiled_vllm_staged is not implemented on this backend "
                       "(a CPU scheduling comparison path)")


bf16_tiled_fused_moe_planned_staged = fused_moe_bf16_tiled_planned_staged
bf16_tiled_fused_moe_vllm_staged = fused_moe_bf16_tiled_vllm_staged


def fused_moe_w8a16_tiled_async_plan(input, weights, topk_weights, topk_ids, plan, *, activation: Any = "silu",
                                     global_num_experts: int = -1, skip_weighted: bool = False, silu_poly_degree: int = 5,
                                     swiglu_limit: float | None = None, cache_dequant: bool = False, out=None):
    """W8A16 forward under an explicit Plan V2 (bf16_tiled.py:1309)."""
    if _fused_moe_w8a16_async_plan_v2_impl is None:
        raise RuntimeError("W8A16 Plan V2 execution is unavailable in this build")
    materialized = plan if isinstance(plan, AsyncMoEPlanV2) else AsyncMoEPlanV2.from_dict(plan)
    if input.dtype != torch.bfloat16:
        raise TypeError("W8A16 input must be a torch.bfloat16 tensor")
    if topk_ids.dtype not in _INTEGER_DTYPES:
        raise TypeError(f"topk_ids must use an integer dtype, got {topk_ids.dtype}")
    if not topk_weights.dtype.is_floating_point:
        raise TypeError(f"topk_weights must use a floating dtype, got {topk_weights.dtype}")
    _validate_output_buffer(input, out)
    result = _fused_moe_w8a16_async_plan_v2_impl(
        input.contiguous(), weights.w13[0], weights.w13[1], weights.w13[2], weights.w13[3], weights.w2[0], weights.w2[1],
        weights.w2[2], weights.w2[3], topk_weights.contiguous(), topk_ids.contiguous(), *_plan_args(materialized),
        materialized.num_threads, _native_activation_name(activation, weights, swiglu_limit), int(global_num_experts),
        bool(skip_weighted), int(silu_poly_degree), int(weights.backend_n_tile), out, materialized.native_early_merge,
        bool(cache_dequant))
    return out if out is not None else result


def fused_moe_w8a16_tiled(input, weights, topk_weights, topk_ids, *, num_threads: int = 1, activation: Any = "silu",
                          global_num_experts: int = -1, skip_weighted: bool = False, silu_poly_degree: int = 5,
                          swiglu_limit: float | None = None, cache_dequant: bool = False, out=None):
    """W8A16 forward through the installed planner runtime (bf16_tiled.py:1380): like W8A8 it has no unplanned path."""
    _require_backend()
    if not isinstance(weights, PreparedW8A16TiledFusedMoEWeights):
        raise TypeError("weights must be PreparedW8A16TiledFusedMoEWeights")
    if input.dtype != torch.bfloat16:
        raise TypeError("W8A16 input must be a torch.bfloat16 tensor")
    if topk_ids.dtype not in _INTEGER_DTYPES:
        raise TypeError(f"topk_ids must use an integer dtype, got {topk_ids.dtype}")
    if not topk_weights.dtype.is_floating_point:
        raise TypeError(f"topk_weights must use a floating dtype, got {topk_weights.dtype}")
    if int(num_threads) <= 0:
        raise ValueError(f"num_threads must be positive, got {num_threads}")
    from .planner_runtime import get_default_moe_planner_runtime

    runtime = get_default_moe_planner_runtime()
    if runtime is None:
        raise RuntimeError("W8A16 fused MoE requires an installed MoePlannerRuntime; "
                           "call enable_moe_planner_quick() or set_default_moe_planner_runtime() first")
    plan = runtime.plan_for_dispatch(weights, topk_ids, num_threads=int(num_threads), activation=activation,
                                     global_num_experts=int(global_num_experts))
    if plan is None:
        raise RuntimeError("the installed MoePlannerRuntime is incompatible with this W8A16 shape, thread count, activation, "
                           "or expert topology")
    return fused_moe_w8a16_tiled_async_plan(input, weights, topk_weights, topk_ids, plan, activation=activation,
                                            global_num_experts=global_num_experts, skip_weighted=skip_weighted,
                                            silu_poly_degree=silu_poly_degree, swiglu_limit=swiglu_limit,
                                            cache_dequant=cache_dequant, out=out)


def fused_moe_w8a8_tiled_async_plan(input, weights, topk_weights, topk_ids, plan, *, activation: Any = "silu",
                                    global_num_experts: int = -1, skip_weighted: bool = False, swiglu_limit: float = 10.0, out=None):
    """W8A8 forward under an explicit Plan V2 (bf16_tiled.py:1450)."""
    if not isinstance(weights, PreparedW8A8TiledFusedMoEWeights):
        raise TypeError("weights must be PreparedW8A8TiledFusedMoEWeights")
    if _fused_moe_w8a8_async_plan_v2_impl is None:
        raise RuntimeError("W8A8 fused MoE Plan V2 requires native fused_moe_w8a8_tiled_async_plan_v2 support")
    if input.dtype != torch.bfloat16:
        raise TypeError("W8A8 input must be a torch.bfloat16 tensor")
    if _activation_name(activation) != "silu" or float(swiglu_limit) != 10.0:
        raise ValueError("W8A8 supports only activation='silu' with swiglu_limit=10.0")
    if topk_ids.dtype not in _INTEGER_DTYPES:
        raise TypeError(f"topk_ids must use an integer dtype, got {topk_ids.dtype}")
    if not topk_weights.dtype.is_floating_point:
        raise TypeError(f"topk_weights must use a floating dtype, got {topk_weights.dtype}")
    _validate_output_buffer(input, out)
    materialized = plan if isinstance(plan, AsyncMoEPlanV2) else AsyncMoEPlanV2.from_dict(plan)
    result = _fused_moe_w8a8_async_plan_v2_impl(
        input.contiguous(), weights.w13[0], weights.w13[1], weights.w13[2], weights.w13[3], weights.w2[0], weights.w2[1],
        weights.w2[2], weights.w2[3], topk_weights.to(torch.float32).contiguous(), topk_ids.to(torch.int64).contiguous(),
        *_plan_args(materialized), materialized.num_threads, "silu", int(global_num_experts), bool(skip_weighted),
        int(weights.backend_n_tile), out, 0, float(swiglu_limit))
    return out if out is not None else result


def fused_moe_w8a8_tiled(input, weights, topk_weights, topk_ids, *, num_threads: int = 1, activation: Any = "silu",
                         global_num_experts: int = -1, skip_weighted: bool = False, swiglu_limit: float = 10.0, out=None):
    """W8A8 forward through the installed planner runtime (bf16_tiled.py:1526)."""
    _require_backend()
    if not isinstance(weights, PreparedW8A8TiledFusedMoEWeights):
        raise TypeError("weights must be PreparedW8A8TiledFusedMoEWeights")
    if int(num_threads) <= 0:
        raise ValueError(f"num_threads must be positive, got {num_threads}")
    from .planner_runtime import get_default_moe_planner_runtime

    runtime = get_default_moe_planner_runtime()
    if runtime is None:
        raise RuntimeError("W8A8 fused MoE requires an installed MoePlannerRuntime; "
                           "call enable_moe_planner_quick() or set_default_moe_planner_runtime() first")
    plan = runtime.plan_for_dispatch(weights, topk_ids, num_threads=int(num_threads), activation=activation,
                                     global_num_experts=int(global_num_experts))
    if plan is None:
        raise RuntimeError("the installed MoePlannerRuntime is incompatible with this W8A8 invocation")
    return fused_moe_w8a8_tiled_async_plan(input, weights, topk_weights, topk_ids, plan, activation=activation,
                                           global_num_experts=global_num_experts, skip_weighted=skip_weighted,
                                           swiglu_limit=swiglu_limit, out=out)


def fused_moe_tiled(input, weights, topk_weights, topk_ids, *, w13_bias=None, w2_bias=None, num_threads: int = 1,
                    activation: Any = "silu", global_num_experts: int = -1, skip_weighted: bool = False,
                    silu_poly_degree: int = 5, swiglu_limit: float | None = None, cache_dequant: bool = False, out=None):
    """Run the implementation selected by the type of the prepared weights (bf16_tiled.py:1576)."""
    common = {"num_threads": num_threads, "activation": activation, "global_num_experts": global_num_experts,
              "skip_weighted": skip_weighted, "silu_poly_degree": silu_poly_degree, "swiglu_limit": swiglu_limit, "out": out}
    if isinstance(weights, PreparedBF16TiledFusedMoEWeights):
        if cache_dequant:
            raise ValueError("cache_dequant is supported only by W8A16 fused MoE weights")
        return fused_moe_bf16_tiled(input, weights, topk_weights, topk_ids, w13_bias=w13_bias, w2_bias=w2_bias, **common)
    if isinstance(weights, PreparedW8A16TiledFusedMoEWeights):
        if w13_bias is not None or w2_bias is not None:
            raise ValueError("W8A16 fused MoE does not support w13_bias or w2_bias")
        return fused_moe_w8a16_tiled(input, weights, topk_weights, topk_ids, cache_dequant=cache_dequant, **common)
    if isinstance(weights, PreparedW8A8TiledFusedMoEWeights):
        if w13_bias is not None or w2_bias is not None:
            raise ValueError("W8A8 fused MoE does not support w13_bias or w2_bias")
        if cache_dequant:
            raise ValueError("cache_dequant is supported only by W8A16 fused MoE weights")
        common.pop("silu_poly_degree")
        return fused_moe_w8a8_tiled(input, weights, topk_weights, topk_ids, **common)
    raise TypeError("weights must be PreparedBF16TiledFusedMoEWeights, PreparedW8A16TiledFusedMoEWeights, "
                    "or PreparedW8A8TiledFusedMoEWeights")


def _combine_with_shared(topk_weights, topk_ids, shared_expert_id: int, scaling: float):
    """Append the shared expert as route K with weight 1 and scale the routed weights (bf16_tiled.py:1007-1013)."""
    tokens, routed_top_k = topk_ids.shape
    ids = torch.empty((tokens, routed_top_k + 1), dtype=topk_ids.dtype, device=topk_ids.device)
    weights = torch.empty((tokens, routed_top_k + 1), dtype=topk_weights.dtype, device=topk_weights.device)
    ids[:, :routed_top_k].copy_(topk_ids)
    ids[:, routed_top_k].fill_(shared_expert_id)
    weights[:, :routed_top_k].copy_(topk_weights * scaling)
    weights[:, routed_top_k].fill_(1.0)
    return weights, ids


def _check_shared_call(input, topk_weights, topk_ids, num_threads, routed_scaling_factor) -> float:
    if input.dtype != torch.bfloat16:
        raise TypeError("input must be a torch.bfloat16 tensor")
    if topk_ids.dtype not in _INTEGER_DTYPES:
        raise TypeError("topk_ids must be an integer tensor")
    if not topk_weights.dtype.is_floating_point:
        raise TypeError("topk_weights must be a floating tensor")
    if topk_ids.dim() != 2 or topk_weights.dim() != 2 or topk_ids.shape != topk_weights.shape:
        raise ValueError("topk_ids and topk_weights must have matching [tokens, top_k] shapes")
    if int(topk_ids.shape[0]) != int(input.shape[0]) or int(topk_ids.shape[1]) <= 0:
        raise ValueError("topk tensors must match input tokens and have positive top_k")
    if int(num_threads) <= 0:
        raise ValueError(f"num_threads must be positive, got {num_threads}")
    scaling = float(routed_scaling_factor)
    if not math.isfinite(scaling):
        raise ValueError("routed_scaling_factor must be finite")
    return scaling


def fused_moe_w8a8_tiled_with_shared(input, weights, topk_weights, topk_ids, *, num_threads: int = 1,
                                     routed_scaling_factor: float = 1.0, activation: Any = "silu", swiglu_limit: float = 10.0,
                                     out=None):
    """W8A8 routed experts plus one always-active shared expert (bf16_tiled.py:964)."""
    _require_backend()
    if not isinstance(weights, PreparedW8A8TiledRoutedSharedMoEWeights):
        raise TypeError("weights must be PreparedW8A8TiledRoutedSharedMoEWeights")
    scaling = _check_shared_call(input, topk_weights, topk_ids, num_threads, routed_scaling_factor)
    if _activation_name(activation) != "silu" or float(swiglu_limit) != 10.0:
        raise ValueError("routed+shared W8A8 requires activation='silu' with swiglu_limit=10.0")
    _validate_output_buffer(input, out)
    combined_weights, combined_ids = _combine_with_shared(topk_weights, topk_ids, weights.shared_expert_id, scaling)
    from .planner_runtime import get_default_moe_planner_runtime

    runtime = get_default_moe_planner_runtime()
    plan = None
    if runtime is not None:
        plan = runtime.plan_for_shared_dispatch(weights, combined_ids, num_threads=int(num_threads), activation="silu")
    if plan is None:
        raise RuntimeError("routed+shared W8A8 fused MoE requires a compatible shared-aware MoePlannerRuntime")
    return fused_moe_w8a8_tiled_async_plan(input, weights.packed, combined_weights, combined_ids, plan, activation="silu",
                                           global_num_experts=-1, swiglu_limit=swiglu_limit, out=out)


def fused_moe_w8a16_tiled_with_shared(input, weights, topk_weights, topk_ids, *, num_threads: int = 1,
                                      routed_scaling_factor: float = 1.0, activation: Any = "silu", silu_poly_degree: int = 5,
                                      swiglu_limit: float | None = None, cache_dequant: bool = False, out=None):
    """W8A16 routed experts plus one always-active shared expert (bf16_tiled.py:881)."""
    _require_backend()
    if not isinstance(weights, PreparedW8A16TiledRoutedSharedMoEWeights):
        raise TypeError("weights must be PreparedW8A16TiledRoutedSharedMoEWeights")
    scaling = _check_shared_call(input, topk_weights, topk_ids, num_threads, routed_scaling_factor)
    _native_activation_name(activation, weights.packed, swiglu_limit)
    if _activation_name(activation) != "silu":
        raise ValueError("routed+shared W8A16 scheduling currently requires activation='silu'")
    _validate_output_buffer(input, out)
    combined_weights, combined_ids = _combine_with_shared(topk_weights, topk_ids, weights.shared_expert_id, scaling)
    from .planner_runtime import get_default_moe_planner_runtime

    runtime = get_default_moe_planner_runtime()
    plan = None
    if runtime is not None:
        plan = runtime.plan_for_shared_dispatch(weights, combined_ids, num_threads=int(num_threads), activation="silu")
    if plan is None:
        raise RuntimeError("routed+shared W8A16 fused MoE requires a compatible shared-aware MoePlannerRuntime")
    return fused_moe_w8a16_tiled_async_plan(input, weights.packed, combined_weights, combined_ids, plan, activation="silu",
                                            global_num_experts=weights.routed_experts + 1, silu_poly_degree=silu_poly_degree,
                                            swiglu_limit=swiglu_limit, cache_dequant=cache_dequant, out=out)


def fused_moe_bf16_tiled_with_shared(input, weights, topk_weights, topk_ids, *, num_threads: int = 1,
                                     routed_scaling_factor: float = 1.0, activation: Any = "silu", silu_poly_degree: int = 5,
                                     swiglu_limit: float | None = None, out=None):
    """BF16 routed experts plus one always-active shared expert (bf16_tiled.py:778)."""
    _require_backend()
    if not isinstance(weights, PreparedBF16TiledRoutedSharedMoEWeights):
        raise TypeError("weights must be PreparedBF16TiledRoutedSharedMoEWeights")
    scaling = _check_shared_call(input, topk_weights, topk_ids, num_threads, routed_scaling_factor)
    if _activation_name(activation) != "silu":
        raise ValueError("routed+shared BF16 scheduling currently requires activation='silu'")
    _validate_output_buffer(input, out)
    combined_weights, combined_ids = _combine_with_shared(topk_weights, topk_ids, weights.shared_expert_id, scaling)
    from .planner_runtime import get_default_moe_planner_runtime

    runtime = get_default_moe_planner_runtime()
    plan = None
    if runtime is not None:
        plan = runtime.plan_for_shared_dispatch(weights, combined_ids, num_threads=int(num_threads), activation="silu")
    if plan is None:
        plan = gpu_placeholder_plan()
    return fused_moe_bf16_tiled_async_plan(input, weights.packed, combined_weights, combined_ids, plan, activation="silu",
                                           silu_poly_degree=silu_poly_degree, swiglu_limit=swiglu_limit, out=out)


def shared_mlp_bf16_tiled(input, weights, *, thread_cpu_ids=None, num_threads: int = 1, silu_poly_degree: int = 5,
                          swiglu_limit: float | None = None, out=None):
    """One prepared expert as a standalone BF16 MLP over every row (bf16_tiled.py:1805): no routing, weight 1."""
    _require_backend()
    if not isinstance(weights, PreparedBF16TiledFusedMoEWeights) or int(weights.w13[0].shape[0]) != 1:
        raise TypeError("weights must be single-expert PreparedBF16TiledFusedMoEWeights")
    tokens = int(input.shape[0])
    ids = torch.zeros((tokens, 1), dtype=torch.int64, device=input.device)
    ones = torch.ones((tokens, 1), dtype=torch.float32, device=input.device)
    return fused_moe_bf16_tiled_async_plan(input, weights, ones, ids, gpu_placeholder_plan(), activation="silu",
                                           silu_poly_degree=silu_poly_degree, swiglu_limit=swiglu_limit, out=out)
