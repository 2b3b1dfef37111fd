"""The op table of the reference's `fused_cpp._moe_C` extension, backed by the B200 C ABI.

Names, positional order and defaults follow the pybind registration in csrc/moe/module.cpp:14-263
(prototypes in csrc/moe/common/api.h:58-162).  Differences that are deliberate:
  * forward ops take CUDA tensors (the reference rejects anything but CPU tensors) and run on the
    current CUDA stream; prepare_* accept CPU or CUDA weights and return CUDA-resident tensors;
  * "packed" weights keep the checkpoint layout [E, N, K]: the tcgen05 kernel reads K-major rows
    through TMA, so there is nothing to repack (the packed objects are opaque by contract,
    docs/public_contracts.md:9-14);
  * Plan V2 placement arrays are checked for consistency and otherwise ignored; the row tiles of the
    two grouped GEMMs ride in task_w13_window_tiles[0] / task_w2_window_tiles[0];
  * ops that only exist as CPU scheduling experiments raise, as unavailable.cpp does on other hosts.
"""
from __future__ import annotations

import os

import torch

from .. import _lib

BACKEND_ID = 200
BACKEND_NAME = "cuda_sm100_tcgen05"
BACKEND_N_TILE = 128
W8A8_BACKEND_NAME = "cuda_sm100_w8a8_tcgen05"


def _device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("fused_cpp_b200 requires a CUDA device (there is no CPU path)")
    return torch.device("cuda", torch.cuda.current_device())


def _numerics() -> int:
    value = os.environ.get("FUSED_CPP_MOE_W8A8_NUMERICS", "torchref").strip().lower()
    if value in ("torchref", "0", ""):
        return _lib.NUMERICS_TORCHREF
    if value in ("native", "1"):
        return _lib.NUMERICS_NATIVE
    raise ValueError("FUSED_CPP_MOE_W8A8_NUMERICS must be 'torchref' or 'native'")


def _gemm_impl() -> int:
    value = os.environ.get("FUSED_CPP_MOE_GEMM_IMPL", "auto").strip().lower()
    table = {"auto": _lib.GEMM_AUTO, "simt": _lib.GEMM_SIMT, "umma": _lib.GEMM_UMMA}
    if value not in table:
        raise ValueError("FUSED_CPP_MOE_GEMM_IMPL must be auto, simt or umma")
    return table[value]


def _route_rows_bf16() -> bool:
    """The reference's opt-in for bf16 route storage, FUSED_CPP_MOE_W2_BF16_ROUTE=1 (default off,
    csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:1016-1019): here it selects the compact route rows of every path
    (fmoe_config.route_rows_bf16): half the bytes of the largest intermediate, output to tolerance instead of bit for bit."""
    return os.environ.get("FUSED_CPP_MOE_W2_BF16_ROUTE", "0") not in ("", "0")


def _sync_check() -> bool:
    return os.environ.get("FUSED_CPP_MOE_SYNC_CHECK", "1") != "0"


def fused_moe_bf16_tiled_available_backends() -> list[str]:
    return [BACKEND_NAME] if _lib.device_supported() else []


def fused_moe_w8a8_tiled_available() -> bool:
    return _lib.device_supported()


def page_policy_info() -> dict:
    return {"backend": BACKEND_NAME, "allocator": "torch caching allocator (cudaMalloc)", "pages": "device"}


def page_mappings() -> list:
    return []


def _check_expert_weights(w13: torch.Tensor, w2: torch.Tensor, dtype: torch.dtype, label: str) -> tuple[int, int, int]:
    if w13.dtype != dtype or w2.dtype != dtype:
        raise RuntimeError(f"{label} weights must have dtype {dtype}")
    if w13.dim() != 3 or w2.dim() != 3:
        raise RuntimeError(f"{label} weights must be [E, 2F, H] and [E, H, F]")
    experts, n13, hidden = w13.shape
    if experts <= 0 or w2.shape[0] != experts:
        raise RuntimeError(f"{label} expert counts must match and be positive")
    if n13 % 2 != 0:
        raise RuntimeError(f"{label} W13 output dimension must be even")
    inter = n13 // 2
    if tuple(w2.shape[1:]) != (hidden, inter):
        raise RuntimeError(f"{label} W2 shape mismatch")
    if hidden % 16 != 0 or inter % 16 != 0:
        raise RuntimeError(f"{label} requires H and F to be multiples of 16")
    return experts, hidden, inter


def fused_moe_bf16_tiled_prepare_weights(w13_weight, w2_weight, fuse_silu=False, backend="auto"):
    """-> (w13_packed, K13, N13, w2_packed, K2, N2, backend_id, n_tile, name); api.h:58-60."""
    if backend not in ("auto", BACKEND_NAME):
        raise RuntimeError(f"unknown BF16 fused MoE backend {backend!r}; available: {BACKEND_NAME}")
    experts, hidden, inter = _check_expert_weights(w13_weight, w2_weight, torch.bfloat16, "BF16 tiled fused MoE")
    device = _device()
    w13 = w13_weight.to(device).contiguous()
    w2 = w2_weight.to(device).contiguous()
    return (w13, hidden, 2 * inter, w2, inter, hidden, BACKEND_ID, BACKEND_N_TILE, BACKEND_NAME)


def fused_moe_bf16_tiled_prepare_routed_shared_weights(routed_w13, routed_w2, shared_w13, shared_w2, backend="auto"):
    """Routed experts followed by the shared expert as expert id E; api.h:72-75."""
    if shared_w13.dim() != 2 or shared_w2.dim() != 2:
        raise RuntimeError("shared weights must be [2F, H] and [H, F]")
    w13 = torch.cat((routed_w13, shared_w13.unsqueeze(0).to(routed_w13.device)), dim=0)
    w2 = torch.cat((routed_w2, shared_w2.unsqueeze(0).to(routed_w2.device)), dim=0)
    return fused_moe_bf16_tiled_prepare_weights(w13, w2, True, backend)


def fused_moe_w8a8_tiled_prepare_quantized_weights(w13_weight, w13_scale, w2_weight, w2_scale):
    """-> (q13, K13, N13, s13[E,2F], q2, K2, N2, s2[E,H], backend_id, n_tile); kernels.cpp:424-444."""
    experts, hidden, inter = _check_expert_weights(w13_weight, w2_weight, torch.int8, "W8A8")
    if w13_scale.dtype != torch.float32 or w2_scale.dtype != torch.float32:
        raise RuntimeError("W8A8 scales must be float32 tensors")
    if w13_scale.numel() != experts * 2 * inter:
        raise RuntimeError("W8A8 W13 scales must contain one value per output channel")
    if w2_scale.numel() != experts * hidden:
        raise RuntimeError("W8A8 W2 scales must contain one value per output channel")
    device = _device()
    return (w13_weight.to(device).contiguous(), hidden, 2 * inter, w13_scale.to(device).reshape(experts, 2 * inter).contiguous(),
            w2_weight.to(device).contiguous(), inter, hidden, w2_scale.to(device).reshape(experts, hidden).contiguous(),
            BACKEND_ID, BACKEND_N_TILE)


def fused_moe_w8a8_tiled_prepare_weights(w13_weight, w2_weight):
    """bf16 weights -> per-output-channel int8 on the GPU, then as above; kernels.cpp:446-461."""
    experts, hidden, inter = _check_expert_weights(w13_weight, w2_weight, torch.bfloat16, "W8A8 source")
    device = _device()
    q13, s13 = _lib.quantize_rows(w13_weight.to(device).reshape(experts * 2 * inter, hidden), weight_mode=True)
    q2, s2 = _lib.quantize_rows(w2_weight.to(device).reshape(experts * hidden, inter), weight_mode=True)
    return fused_moe_w8a8_tiled_prepare_quantized_weights(q13.reshape(experts, 2 * inter, hidden), s13.reshape(experts, 2 * inter),
                                                          q2.reshape(experts, hidden, inter), s2.reshape(experts, hidden))


def _check_out(input: torch.Tensor, out: torch.Tensor | None, others) -> None:
    if out is None:
        return
    if out.device != input.device or out.dtype != torch.bfloat16 or out.shape != input.shape or not out.is_contiguous():
        raise RuntimeError("out must be a contiguous BF16 tensor with the input shape on the input's device")
    if out.requires_grad:
        raise RuntimeError("out with requires_grad=True is not supported")
    for other in others:
        if other is not None and out.untyped_storage().data_ptr() == other.untyped_storage().data_ptr():
            raise RuntimeError("out must not alias the input, weights or top-k tensors")


def _tile_from(windows) -> int:
    if windows is None or windows.numel() == 0:
        return 0
    return int(windows.reshape(-1)[0])


def _check_plan_vectors(task_expert_ids, task_core_begins, task_threads, task_dep_offsets, task_deps, plan_version,
                        execution_mode, task_min_threads, task_max_threads, task_resize_points, label):
    if plan_version != 2 or execution_mode != 0:
        raise RuntimeError(f"{label} requires strict Plan V2 execution")
    tasks = task_expert_ids.numel()
    for tensor in (task_core_begins, task_threads, task_min_threads, task_max_threads):
        if tensor.numel() != tasks:
            raise RuntimeError(f"{label} task vectors must have matching lengths")
    if task_dep_offsets.numel() != tasks + 1 or int(task_dep_offsets[tasks]) != task_deps.numel():
        raise RuntimeError(f"{label} dependency offsets are invalid")
    if task_resize_points.numel() and bool((task_resize_points != 0).any()):
        raise RuntimeError(f"{label} does not support dynamic resize points")


def fused_moe_w8a8_tiled_async_plan_v2(
        input, w13_packed, w13_k, w13_n, w13_scales, w2_packed, w2_k, w2_n, w2_scales, topk_weights, topk_ids,
        task_expert_ids, task_core_begins, task_threads, task_dep_offsets, task_deps, plan_version, execution_mode,
        task_preferred_threads, task_min_threads, task_max_threads, task_allowed_thread_offsets, task_allowed_threads,
        task_placement_modes, task_numa_nodes, task_stage_ids, task_resize_points, task_range_granularities,
        task_w13_window_tiles=None, task_w2_window_tiles=None, thread_cpu_ids=None, num_threads=1, activation="silu",
        global_num_experts=-1, skip_weighted=False, backend_n_tile=8, out=None, early_merge=0, swiglu_limit=10.0):
    """The W8A8 forward op; csrc/moe/module.cpp:205-220, csrc/moe/arm/i8mm_w8a8/kernels.cpp:463-694."""
    _check_plan_vectors(task_expert_ids, task_core_begins, task_threads, task_dep_offsets, task_deps, plan_version,
                        execution_mode, task_min_threads, task_max_threads, task_resize_points, "W8A8")
    if activation != "silu" or float(swiglu_limit) != 10.0:
        raise RuntimeError("W8A8 supports only clamped SwiGLU limit 10.0")
    if global_num_experts != -1:
        raise RuntimeError("W8A8 v1 does not support expert-parallel id remapping")
    if skip_weighted:
        raise RuntimeError("W8A8 v1 requires weighted TopK merge")
    if early_merge != 0:
        raise RuntimeError("W8A8 v1 requires early_merge=False")
    if input.dim() != 2 or input.dtype != torch.bfloat16 or input.device.type != "cuda":
        raise RuntimeError("W8A8 input must be a CUDA BF16 [tokens, H] tensor")
    if topk_ids.dim() != 2 or topk_weights.shape != topk_ids.shape or topk_ids.shape[0] != input.shape[0]:
        raise RuntimeError("W8A8 topk tensors must be matching [tokens, top_k]")
    if topk_ids.dtype != torch.int64:
        raise RuntimeError("W8A8 topk_ids must be torch.int64")
    if topk_weights.dtype != torch.float32:
        raise RuntimeError("W8A8 topk_weights must be torch.float32")
    if input.shape[1] != w13_k or w13_n != 2 * w2_k or w2_n != w13_k:
        raise RuntimeError("W8A8 expert dimensions mismatch")
    if backend_n_tile != BACKEND_N_TILE:
        raise RuntimeError("W8A8 backend N tile mismatch")
    experts = w13_packed.shape[0]
    if tuple(w13_scales.shape) != (experts, w13_n) or tuple(w2_scales.shape) != (experts, w2_n):
        raise RuntimeError("W8A8 scale shapes are invalid")
    _check_out(input, out, (input, w13_packed, w2_packed, topk_weights, topk_ids))
    w13 = w13_packed.reshape(experts, w13_n, w13_k)
    w2 = w2_packed.reshape(experts, w2_n, w2_k)
    result = _lib.moe_forward(input, w13, w2, topk_weights, topk_ids, s13=w13_scales, s2=w2_scales, numerics=_numerics(),
                              gemm_impl=_gemm_impl(), gate_up_tile=_tile_from(task_w13_window_tiles),
                              down_tile=_tile_from(task_w2_window_tiles), swiglu_limit=float(swiglu_limit), out=out,
                              route_rows_bf16=_route_rows_bf16())
    if _sync_check():
        result.raise_for_status()
    if out is not None:
        out._version  # noqa: B018  (written in place by the kernels; torch tracks no version bump for raw pointers)
    return result.out


def _native_activation(activation: str) -> tuple[int, float]:
    """Activation string of the op -> (activation id of the C ABI, swiglu_limit)."""
    table = {"silu": (_lib.ACTIVATION_SILU, 0.0), "silu_clamp10": (_lib.ACTIVATION_SILU, 10.0),
             "gelu": (_lib.ACTIVATION_GELU, 0.0), "swigluoai": (_lib.ACTIVATION_SWIGLUOAI, 0.0)}
    if activation not in table:
        raise RuntimeError(f"unsupported MoE activation: {activation}")
    return table[activation]


def _check_bias(bias, experts: int, channels: int, name: str):
    """check_optional_bias of the reference (fused_moe_bf16_tiled.cpp:6420-6421): [E, N] of a floating dtype."""
    if bias is None:
        return None
    if bias.dim() != 2 or tuple(bias.shape) != (experts, channels) or not bias.dtype.is_floating_point:
        raise RuntimeError(f"{name} must be a floating [E, N] = [{experts}, {channels}] tensor")
    return bias.to(device=_device(), dtype=torch.float32).contiguous()


# swigluoai checkpoints interleave gate and up channels (row 2j = gate j, row 2j + 1 = up j; naive.py:39-47); the
# kernels take gate rows then up rows.  The reordered copy is made once per weight tensor and kept while it lives.
_DEINTERLEAVED: dict = {}


def _gate_then_up(tensor: torch.Tensor, dim: int) -> torch.Tensor:
    key = (tensor.data_ptr(), tuple(tensor.shape), tensor.dtype, dim)
    cached = _DEINTERLEAVED.get(key)
    if cached is not None and cached[0]() is tensor:
        return cached[1]
    import weakref

    count = tensor.shape[dim]
    order = torch.cat((torch.arange(0, count, 2), torch.arange(1, count, 2))).to(tensor.device)
    result = tensor.index_select(dim, order).contiguous()
    for stale in [k for k, v in _DEINTERLEAVED.items() if v[0]() is None]:
        del _DEINTERLEAVED[stale]
    _DEINTERLEAVED[key] = (weakref.ref(tensor), result)
    return result


def _bf16_forward(input, w13_packed, w13_k, w13_n, w2_packed, w2_k, w2_n, topk_weights, topk_ids, w13_bias, w2_bias,
                  activation, global_num_experts, skip_weighted, out, gate_up_tile=0, down_tile=0):
    if input.dim() != 2 or input.dtype != torch.bfloat16 or input.device.type != "cuda":
        raise RuntimeError("input must be a CUDA BF16 [tokens, H] tensor")
    if topk_ids.dim() != 2 or topk_weights.shape != topk_ids.shape or topk_ids.shape[0] != input.shape[0]:
        raise RuntimeError("topk tensors must be matching [tokens, top_k]")
    if input.shape[1] != w13_k or w13_n != 2 * w2_k or w2_n != w13_k:
        raise RuntimeError("expert dimensions mismatch")
    experts = w13_packed.shape[0]
    if global_num_experts == 0 or global_num_experts < -1:
        raise RuntimeError(f"global_num_experts must be positive or -1, got {global_num_experts}")
    if global_num_experts != -1 and global_num_experts > experts:
        raise RuntimeError("global_num_experts cannot exceed the packed expert count")
    if skip_weighted and topk_ids.shape[1] != 1:
        raise RuntimeError("skip_weighted is only valid when top_k == 1")
    _check_out(input, out, (input, w13_packed, w2_packed, topk_weights, topk_ids))
    activation_id, limit = _native_activation(activation)
    w13_bias = _check_bias(w13_bias, experts, w13_n, "w13_bias")
    w2_bias = _check_bias(w2_bias, experts, w2_n, "w2_bias")
    w13 = w13_packed.reshape(experts, w13_n, w13_k)
    w2 = w2_packed.reshape(experts, w2_n, w2_k)
    if activation_id == _lib.ACTIVATION_SWIGLUOAI:
        w13 = _gate_then_up(w13, 1)
        if w13_bias is not None:
            w13_bias = _gate_then_up(w13_bias, 1)
    # The reference narrows the valid id range to [0, global_num_experts) and raises on ids beyond it
    # (fused_moe_bf16_tiled.cpp:6439-6458): the route build sees only that many experts, so such ids are reported as
    # out of range instead of being routed to the trailing prepared experts.
    if global_num_experts != -1 and global_num_experts < experts:
        experts = int(global_num_experts)
        w13, w2 = w13[:experts], w2[:experts]
        w13_bias = None if w13_bias is None else w13_bias[:experts]
        w2_bias = None if w2_bias is None else w2_bias[:experts]
    weights = topk_weights.to(torch.float32)
    if skip_weighted:
        weights = torch.ones_like(weights)
    result = _lib.moe_forward(input, w13, w2, weights, topk_ids.to(torch.int64), gemm_impl=_gemm_impl(), gate_up_tile=gate_up_tile,
                              down_tile=down_tile, swiglu_limit=limit, out=out, activation=activation_id, w13_bias=w13_bias,
                              w2_bias=w2_bias, route_rows_bf16=_route_rows_bf16())
    if _sync_check():
        result.raise_for_status()
    return result.out


def fused_moe_bf16_tiled(input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, topk_weights, topk_ids, w13_bias=None,
                         w2_bias=None, num_threads=1, activation="silu", global_num_experts=-1, skip_weighted=False,
                         fuse_silu=False, silu_poly_degree=5, gemm_backend=0, backend_n_tile=8, out=None):
    """The BF16 forward op; csrc/moe/module.cpp:132-139, fused_moe_bf16_tiled.cpp:6376."""
    if silu_poly_degree not in (4, 5, 6):
        raise RuntimeError("silu_poly_degree must be 4, 5 or 6")
    return _bf16_forward(input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, topk_weights, topk_ids, w13_bias, w2_bias,
                         activation, global_num_experts, skip_weighted, out)


def fused_moe_bf16_tiled_async_plan_v2(
        input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, topk_weights, topk_ids, task_expert_ids, task_core_begins,
        task_threads, task_dep_offsets, task_deps, plan_version, execution_mode, task_preferred_threads, task_min_threads,
        task_max_threads, task_allowed_thread_offsets, task_allowed_threads, task_placement_modes, task_numa_nodes,
        task_stage_ids, task_resize_points, task_range_granularities, task_w13_window_tiles=None, task_w2_window_tiles=None,
        thread_cpu_ids=None, w13_bias=None, w2_bias=None, num_threads=1, activation="silu", global_num_experts=-1,
        skip_weighted=False, fuse_silu=False, silu_poly_degree=5, gemm_backend=0, backend_n_tile=8, out=None, early_merge=-1):
    """The BF16 Plan V2 op; csrc/moe/module.cpp:162-177, fused_moe_bf16_tiled.cpp:9394."""
    if plan_version != 2:
        raise RuntimeError("BF16 async plan requires plan_version 2")
    return _bf16_forward(input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, topk_weights, topk_ids, w13_bias, w2_bias,
                         activation, global_num_experts, skip_weighted, out, _tile_from(task_w13_window_tiles),
                         _tile_from(task_w2_window_tiles))


def fused_moe_bf16_tiled_scheduled(input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, topk_weights, topk_ids,
                                   wave_offsets, team_expert_ids, team_threads, thread_cpu_ids=None, w13_bias=None,
                                   w2_bias=None, num_threads=1, activation="silu", global_num_experts=-1, skip_weighted=False,
                                   fuse_silu=False, silu_poly_degree=5, gemm_backend=0, backend_n_tile=8, out=None):
    """Wave/team schedule variant (csrc/moe/module.cpp:141-150): the CPU placement is ignored on the GPU."""
    return _bf16_forward(input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, topk_weights, topk_ids, w13_bias, w2_bias,
                         activation, global_num_experts, skip_weighted, out)


def fused_moe_bf16_tiled_async(input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, topk_weights, topk_ids,
                               task_expert_ids, task_core_begins, task_threads, task_dep_offsets, task_deps,
                               thread_cpu_ids=None, w13_bias=None, w2_bias=None, num_threads=1, activation="silu",
                               global_num_experts=-1, skip_weighted=False, fuse_silu=False, silu_poly_degree=5,
                               gemm_backend=0, backend_n_tile=8, out=None):
    """Async task-DAG variant (csrc/moe/module.cpp:152-160): the CPU task graph is ignored on the GPU."""
    return _bf16_forward(input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, topk_weights, topk_ids, w13_bias, w2_bias,
                         activation, global_num_experts, skip_weighted, out)


def shared_mlp_bf16_tiled(input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, thread_cpu_ids=None, num_threads=1,
                          fuse_silu=True, silu_poly_degree=5, gemm_backend=1, backend_n_tile=8, out=None, clamp_swiglu=False):
    """One packed BF16 expert as a standalone MLP over every row (csrc/moe/module.cpp:244-250, api.h:158-162):
    no routing, every row goes to expert 0 with weight 1."""
    if w13_packed.dim() != 3 or int(w13_packed.shape[0]) != 1:
        raise RuntimeError("shared_mlp_bf16_tiled expects a single-expert packed weight")
    if input.dim() != 2:
        raise RuntimeError("input must be a [tokens, H] tensor")
    tokens = int(input.shape[0])
    ids = torch.zeros((tokens, 1), dtype=torch.int64, device=input.device)
    ones = torch.ones((tokens, 1), dtype=torch.float32, device=input.device)
    return _bf16_forward(input, w13_packed, w13_K, w13_N, w2_packed, w2_K, w2_N, ones, ids, None, None,
                         "silu_clamp10" if clamp_swiglu else "silu", -1, False, out)


class NativeQuickPlanner:
    """Greedy longest-first lane assignment over homogeneous team shapes: the class the reference's Python planner
    looks up in `fused_cpp._moe_C` (csrc/moe_planner/quick_bindings.cpp:120-132; behaviour of
    csrc/moe_planner/interval_planner.cpp:1616-1870).  Costs come from the caller's model as plain floats.

    A shape is a list of equal team widths that sum to num_cores; a lane is one team.  Experts are taken in
    descending route count (stable), each goes to the lane whose load after adding the expert's cost is smallest,
    ties to the lower lane index.  `plan` scores every configured shape and keeps the smallest makespan (ties:
    working-set bytes, then lanes); `plan_shared` pins the synthetic shared expert to lane 0 first and accepts
    shapes of mixed widths with one cost row per width.  On the GPU build nothing consumes the CPU placement that
    comes out; the class exists so that the planner tool chain keeps working against this package.
    """

    def __init__(self, num_cores, shapes, max_stage_bytes, window_bytes_by_width, relative_error, profile_runs=1,
                 planner_threads=1):
        self._cores = int(num_cores)
        self._shapes = [[int(w) for w in shape] for shape in shapes]
        self._stage_bytes = int(max_stage_bytes)
        self._window = {int(width): int(nbytes) for width, nbytes in window_bytes_by_width}
        self._relative_error = float(relative_error)
        self._profile_runs = int(profile_runs)
        if self._cores <= 0 or self._stage_bytes <= 0 or self._profile_runs <= 0:
            raise ValueError("native quick planner dimensions and profile_runs must be positive")
        if int(planner_threads) < 0:
            raise ValueError("native quick planner threads must be non-negative")
        workers = int(planner_threads) if int(planner_threads) > 0 else min(8, self._cores, os.cpu_count() or self._cores)
        self._workers = max(1, min(workers, self._cores))
        if not (self._relative_error >= 0.0) or self._relative_error == float("inf"):
            raise ValueError("native quick planner relative_error must be finite and non-negative")
        if not self._shapes:
            raise ValueError("native quick planner requires homogeneous shapes")
        for shape in self._shapes:
            if not self._homogeneous(shape):
                raise ValueError("native quick planner shapes must be homogeneous and cover num_cores")
            if self._window.get(shape[0], 0) <= 0:
                raise ValueError("native quick planner is missing positive window bytes for a shape width")

    @property
    def configured_workers(self) -> int:
        return self._workers

    def _homogeneous(self, shape) -> bool:
        return bool(shape) and sum(shape) == self._cores and all(width == shape[0] for width in shape)

    def _candidate(self, shape, lanes, loads, expert_ids, routes, windows) -> dict:
        makespan = max(loads)
        waves = max(1, -(-len(routes) // len(shape)))
        uncertainty = makespan * self._relative_error / float(waves * self._profile_runs) ** 0.5
        tasks = []
        core_begin = 0
        for lane, members in enumerate(lanes):
            previous = -1
            for index in members:
                tasks.append((int(expert_ids[index]), int(routes[index]), core_begin, int(shape[lane]), [previous] if previous >= 0 else []))
                previous = len(tasks) - 1
            core_begin += int(shape[lane])
        return {"shape": list(shape), "assignment_order": "lpt", "execution_mode": "strict", "tail_pool_threads": None,
                "tail_pool_max_routes": None, "tail_pool_tasks": 0, "tail_repartition_width": None, "tail_repartition_tasks": 0,
                "tail_repartition_route_slices": 1, "makespan_ns": makespan, "uncertainty_ns": uncertainty,
                "pessimistic_ns": makespan + uncertainty, "tasks": tasks,
                "active_working_set_bytes": len(shape) * self._stage_bytes, "window_bytes_per_worker": list(windows),
                "resource_groups": len(shape)}

    @staticmethod
    def _descending_by_routes(routes, skip=None):
        return sorted((i for i in range(len(routes)) if i != skip), key=lambda i: -routes[i])  # sorted() is stable

    def assign(self, expert_ids, routes, shape, costs) -> dict:
        expert_ids, routes, shape = list(expert_ids), [int(r) for r in routes], [int(w) for w in shape]
        costs = [float(c) for c in costs]
        if not expert_ids or len(expert_ids) != len(routes) or len(routes) != len(costs):
            raise ValueError("native quick planner expert_ids, routes, and costs must have equal positive size")
        if not self._homogeneous(shape):
            raise ValueError("native quick assignment requires a homogeneous shape covering num_cores")
        if any(r <= 0 for r in routes) or any(not (0.0 < c < float("inf")) for c in costs):
            raise ValueError("native quick planner routes and costs must be positive and finite")
        if shape[0] not in self._window:
            raise ValueError("native quick planner is missing window bytes for assignment width")
        loads = [0.0] * len(shape)
        lanes = [[] for _ in shape]
        for index in self._descending_by_routes(routes):
            # Smallest resulting load; among equal sums (after rounding) the lowest lane.
            best = min(range(len(shape)), key=lambda lane: (loads[lane] + costs[index], lane))
            lanes[best].append(index)
            loads[best] += costs[index]
        return self._candidate(shape, lanes, loads, expert_ids, routes, [self._window[shape[0]]] * len(shape))

    def _assign_shared(self, expert_ids, routes, shared_expert_id, shape, cost_rows) -> dict:
        if not shape or sum(shape) != self._cores:
            raise ValueError("native shared quick shape must cover num_cores")
        for width in shape:
            if width <= 0 or width not in cost_rows:
                raise ValueError("native shared quick shape width is missing a cost row")
            if width not in self._window:
                raise ValueError("native shared quick shape width is missing window bytes")
        if expert_ids.count(shared_expert_id) != 1:
            raise ValueError("native shared quick planner requires exactly one synthetic shared expert")
        shared = expert_ids.index(shared_expert_id)
        loads = [0.0] * len(shape)
        lanes = [[] for _ in shape]
        lanes[0].append(shared)
        loads[0] = cost_rows[shape[0]][shared]
        for index in self._descending_by_routes(routes, skip=shared):
            best = min(range(len(shape)), key=lambda lane: (loads[lane] + cost_rows[shape[lane]][index], lane))
            loads[best] += cost_rows[shape[best]][index]
            lanes[best].append(index)
        return self._candidate(shape, lanes, loads, expert_ids, routes, [self._window[w] for w in shape])

    @staticmethod
    def _select_with_uncertainty(candidates) -> dict:
        """Among the candidates whose uncertainty band overlaps the fastest one's, the smallest working set, then
        the fewest lanes, then the smaller pessimistic time (interval_planner.cpp:150-172)."""
        ordered = sorted(candidates, key=lambda c: c["makespan_ns"])
        fastest = ordered[0]
        low, high = fastest["makespan_ns"] - fastest["uncertainty_ns"], fastest["pessimistic_ns"]
        overlapping = [c for c in ordered if c["makespan_ns"] - c["uncertainty_ns"] <= high and c["pessimistic_ns"] >= low]
        return min(overlapping, key=lambda c: (c["active_working_set_bytes"], c["resource_groups"], 0, c["pessimistic_ns"], c["makespan_ns"]))

    def _result(self, candidates, selected) -> dict:
        return {"selected": selected, "candidates": [{k: v for k, v in c.items() if k != "tasks"} for c in candidates],
                "configured_workers": self._workers, "strict_candidates": len(candidates)}

    def plan(self, expert_ids, routes, costs) -> dict:
        costs = [list(row) for row in costs]
        if len(costs) != len(self._shapes):
            raise ValueError("native quick planner requires one cost row per shape")
        candidates = [self.assign(expert_ids, routes, shape, row) for shape, row in zip(self._shapes, costs)]
        selected = min(candidates, key=lambda c: (c["makespan_ns"], c["active_working_set_bytes"], c["resource_groups"]))
        return self._result(candidates, selected)

    def plan_shared(self, expert_ids, routes, shared_expert_id, shapes, cost_widths, costs_by_width) -> dict:
        expert_ids, routes = list(expert_ids), [int(r) for r in routes]
        shapes = [[int(w) for w in shape] for shape in shapes]
        if not shapes:
            raise ValueError("native shared quick planner requires candidate shapes")
        if not expert_ids or len(expert_ids) != len(routes) or len(cost_widths) != len(costs_by_width):
            raise ValueError("native shared quick planner inputs must have matching positive sizes")
        cost_rows: dict = {}
        for width, row in zip(cost_widths, costs_by_width):
            if int(width) <= 0 or len(row) != len(routes) or int(width) in cost_rows:
                raise ValueError("native shared quick cost rows must have unique positive widths and expert costs")
            cost_rows[int(width)] = [float(c) for c in row]
        candidates = [self._assign_shared(expert_ids, routes, int(shared_expert_id), shape, cost_rows) for shape in shapes]
        # The selection sorts by makespan first; the candidate list is returned in that order, as the reference's is.
        candidates.sort(key=lambda c: c["makespan_ns"])
        return self._result(candidates, self._select_with_uncertainty(candidates))


def _not_built(name: str, why: str):
    def raiser(*_args, **_kwargs):
        raise RuntimeError(f"{name} is not implemented on this backend: {why}")
    raiser.__name__ = name
    return raiser


_CPU_ONLY = "it is a CPU thread-scheduling experiment; use fused_moe_bf16_tiled or fused_moe_bf16_tiled_async_plan_v2"
fused_moe_bf16_tiled_planned_staged = _not_built("fused_moe_bf16_tiled_planned_staged", _CPU_ONLY)
fused_moe_bf16_tiled_vllm_staged = _not_built("fused_moe_bf16_tiled_vllm_staged", _CPU_ONLY)


# ---- W8A16: int8 weights + per-output-channel scales, bf16 activations --------------------------------------

W8A16_BACKEND_NAME = "cuda_sm100_w8a16_tcgen05"


def fused_moe_w8a16_tiled_prepare_quantized_weights(w13_weight, w13_scale, w2_weight, w2_scale):
    """Checkpoint int8 weights + scales -> (q13, K13, N13, s13[E,2F], q2, K2, N2, s2[E,H], backend_id, n_tile) on the GPU
    (api.h:64-66).  The layout and the checks are those of the W8A8 preparation: both paths read the same tensors."""
    return fused_moe_w8a8_tiled_prepare_quantized_weights(w13_weight, w13_scale, w2_weight, w2_scale)


def fused_moe_w8a16_tiled_prepare_weights(w13_weight, w2_weight):
    """bf16 weights -> symmetric per-output-channel int8 (scale = amax / 127, round to nearest even, clamp +-127:
    quantize_pack_expert_weight_per_channel, fused_moe_bf16_tiled.cpp:4950-4976), api.h:61-62."""
    return fused_moe_w8a8_tiled_prepare_weights(w13_weight, w2_weight)


def fused_moe_w8a16_tiled_prepare_quantized_routed_shared_weights(routed_w13_weight, routed_w13_scale, routed_w2_weight,
                                                                  routed_w2_scale, shared_w13_weight, shared_w13_scale,
                                                                  shared_w2_weight, shared_w2_scale):
    """Routed experts followed by the shared expert as expert id E (api.h:67-71)."""
    if shared_w13_weight.dim() != 2 or shared_w2_weight.dim() != 2:
        raise RuntimeError("shared W8A16 weights must be [2F, H] and [H, F]")
    experts = routed_w13_weight.shape[0]
    return fused_moe_w8a16_tiled_prepare_quantized_weights(
        torch.cat((routed_w13_weight, shared_w13_weight.unsqueeze(0).to(routed_w13_weight.device)), dim=0),
        torch.cat((routed_w13_scale.reshape(experts, -1), shared_w13_scale.reshape(1, -1).to(routed_w13_scale.device)), dim=0),
        torch.cat((routed_w2_weight, shared_w2_weight.unsqueeze(0).to(routed_w2_weight.device)), dim=0),
        torch.cat((routed_w2_scale.reshape(experts, -1), shared_w2_scale.reshape(1, -1).to(routed_w2_scale.device)), dim=0))


def fused_moe_w8a16_tiled_async_plan_v2(
        input, w13_packed, w13_K, w13_N, w13_scales, w2_packed, w2_K, w2_N, w2_scales, topk_weights, topk_ids,
        task_expert_ids, task_core_begins, task_threads, task_dep_offsets, task_deps, plan_version, execution_mode,
        task_preferred_threads, task_min_threads, task_max_threads, task_allowed_thread_offsets, task_allowed_threads,
        task_placement_modes, task_numa_nodes, task_stage_ids, task_resize_points, task_range_granularities,
        task_w13_window_tiles=None, task_w2_window_tiles=None, thread_cpu_ids=None, num_threads=1, activation="silu",
        global_num_experts=-1, skip_weighted=False, silu_poly_degree=5, backend_n_tile=8, out=None, early_merge=-1,
        cache_dequant=False):
    """The W8A16 forward op (csrc/moe/module.cpp:180-194).  cache_dequant is accepted and has no effect: it selects
    the reference's cached bf16 copy of a weight window, a CPU cache-blocking device; here the int8 weights meet the
    activations as they lie in memory (activations as 16-bit fixed point per row on the int8 tensor cores, or, with
    FUSED_CPP_MOE_W8A16_FORM=bf16, bf16 activations against weight tiles widened in shared memory) and the per-channel
    scale multiplies the accumulator."""
    if plan_version != 2:
        raise RuntimeError("W8A16 async plan requires plan_version 2")
    if input.dim() != 2 or input.dtype != torch.bfloat16 or input.device.type != "cuda":
        raise RuntimeError("W8A16 input must be a CUDA BF16 [tokens, H] tensor")
    if topk_ids.dim() != 2 or topk_weights.shape != topk_ids.shape or topk_ids.shape[0] != input.shape[0]:
        raise RuntimeError("W8A16 topk tensors must be matching [tokens, top_k]")
    if input.shape[1] != w13_K or w13_N != 2 * w2_K or w2_N != w13_K:
        raise RuntimeError("W8A16 expert dimensions mismatch")
    if w13_packed.dtype != torch.int8 or w2_packed.dtype != torch.int8:
        raise RuntimeError("W8A16 packed weights must be int8")
    experts = int(w13_packed.shape[0])
    if tuple(w13_scales.shape) != (experts, w13_N) or tuple(w2_scales.shape) != (experts, w2_N):
        raise RuntimeError("W8A16 scale shapes are invalid")
    if global_num_experts == 0 or global_num_experts < -1 or global_num_experts > experts:
        raise RuntimeError("global_num_experts must be -1 or in [1, prepared experts]")
    if skip_weighted and topk_ids.shape[1] != 1:
        raise RuntimeError("skip_weighted is only valid when top_k == 1")
    if silu_poly_degree not in (4, 5, 6):
        raise RuntimeError("silu_poly_degree must be 4, 5 or 6")
    _check_out(input, out, (input, w13_packed, w2_packed, topk_weights, topk_ids))
    activation_id, limit = _native_activation(activation)
    w13 = w13_packed.reshape(experts, w13_N, w13_K)
    w2 = w2_packed.reshape(experts, w2_N, w2_K)
    s13, s2 = w13_scales, w2_scales
    if activation_id == _lib.ACTIVATION_SWIGLUOAI:
        w13, s13 = _gate_then_up(w13, 1), _gate_then_up(s13, 1)
    if global_num_experts != -1 and global_num_experts < experts:
        experts = int(global_num_experts)
        w13, w2, s13, s2 = w13[:experts], w2[:experts], s13[:experts], s2[:experts]
    weights = topk_weights.to(torch.float32)
    if skip_weighted:
        weights = torch.ones_like(weights)
    result = _lib.moe_forward(input, w13, w2, weights, topk_ids.to(torch.int64), s13=s13.contiguous(), s2=s2.contiguous(), w8a16=True,
                              gate_up_tile=_tile_from(task_w13_window_tiles), down_tile=_tile_from(task_w2_window_tiles),
                              swiglu_limit=limit, out=out, activation=activation_id, route_rows_bf16=_route_rows_bf16())
    if _sync_check():
        result.raise_for_status()
    return result.out
