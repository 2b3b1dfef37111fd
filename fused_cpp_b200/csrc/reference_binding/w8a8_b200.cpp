// The binding a maintainer of the reference would add on a CUDA build: the body of the reference's
// fused_moe_w8a8_tiled_async_plan_v2 (csrc/moe/arm/i8mm_w8a8/kernels.cpp:463-694; prototype csrc/moe/common/api.h:131-142;
// pybind registration csrc/moe/module.cpp:205-220, which stays as it is) expressed over the C ABI of
// libfused_moe_b200.so.  at::Tensor arguments are unwrapped into device pointers, the caller's CUDA stream is passed
// through, errors become TORCH_CHECK failures (RuntimeError in Python), as everywhere in the reference.
//
// This file is not part of the library (which has no torch dependency).  It is compiled against the torch headers by
// tests/test_reference_binding.py so that the text shown in INTEGRATION.md is known to be valid C++.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/util/Optional.h>

#include <string>

#include "fused_moe_b200.h"

namespace {

// First element of an optional int64 CPU tensor (the Plan V2 window fields), 0 when absent or empty.
int first_or_zero(const c10::optional<at::Tensor>& values) {
  if (!values.has_value() || values->numel() == 0) return 0;
  return static_cast<int>(values->reshape({-1})[0].item<int64_t>());
}

}  // namespace

at::Tensor fused_moe_w8a8_tiled_async_plan_v2(
    at::Tensor input, at::Tensor w13_packed, int64_t w13_K, int64_t w13_N, at::Tensor w13_scales, at::Tensor w2_packed,
    int64_t w2_K, int64_t w2_N, at::Tensor w2_scales, at::Tensor topk_weights, at::Tensor topk_ids,
    at::Tensor task_expert_ids, at::Tensor task_core_begins, at::Tensor task_threads, at::Tensor task_dep_offsets,
    at::Tensor task_deps, int64_t plan_version, int64_t execution_mode, at::Tensor task_preferred_threads,
    at::Tensor task_min_threads, at::Tensor task_max_threads, at::Tensor task_allowed_thread_offsets,
    at::Tensor task_allowed_threads, at::Tensor task_placement_modes, at::Tensor task_numa_nodes, at::Tensor task_stage_ids,
    at::Tensor task_resize_points, at::Tensor task_range_granularities, c10::optional<at::Tensor> task_w13_window_tiles,
    c10::optional<at::Tensor> task_w2_window_tiles, c10::optional<at::Tensor> thread_cpu_ids, int64_t num_threads,
    std::string activation, int64_t global_num_experts, bool skip_weighted, int64_t backend_n_tile,
    c10::optional<at::Tensor> out, int64_t early_merge, double swiglu_limit) {
  // The CPU placement of the plan (cores, threads, NUMA nodes, dependencies) has no meaning on the GPU: the plan must
  // be a well-formed strict Plan V2, its two window fields carry the row tiles of the grouped GEMMs (0 = automatic).
  TORCH_CHECK(plan_version == 2 && execution_mode == 0, "W8A8 requires strict Plan V2 execution");
  const int64_t tasks = task_expert_ids.numel();
  TORCH_CHECK(task_core_begins.numel() == tasks && task_threads.numel() == tasks && task_min_threads.numel() == tasks &&
                  task_max_threads.numel() == tasks && task_preferred_threads.numel() == tasks,
              "W8A8 task vectors must have matching lengths");
  TORCH_CHECK(task_dep_offsets.numel() == tasks + 1 && task_dep_offsets[tasks].item<int64_t>() == task_deps.numel(),
              "W8A8 dependency offsets are invalid");
  (void)task_allowed_thread_offsets, (void)task_allowed_threads, (void)task_placement_modes, (void)task_numa_nodes;
  (void)task_stage_ids, (void)task_resize_points, (void)task_range_granularities, (void)thread_cpu_ids, (void)num_threads;
  TORCH_CHECK(activation == "silu" && swiglu_limit == 10.0, "W8A8 supports only clamped SwiGLU limit 10.0");
  TORCH_CHECK(global_num_experts == -1, "W8A8 v1 does not support expert-parallel id remapping");
  TORCH_CHECK(!skip_weighted, "W8A8 v1 requires weighted TopK merge");
  TORCH_CHECK(early_merge == 0, "W8A8 v1 requires early_merge=False");
  (void)backend_n_tile;

  TORCH_CHECK(input.is_cuda() && input.dim() == 2 && input.scalar_type() == at::kBFloat16 && input.is_contiguous(),
              "W8A8 input must be a contiguous CUDA BF16 [tokens, H] tensor");
  TORCH_CHECK(topk_ids.scalar_type() == at::kLong && topk_weights.scalar_type() == at::kFloat && topk_ids.dim() == 2 &&
                  topk_weights.sizes() == topk_ids.sizes() && topk_ids.size(0) == input.size(0),
              "W8A8 topk tensors must be matching [tokens, top_k] (int64 ids, float32 weights)");
  TORCH_CHECK(input.size(1) == w13_K && w13_N == 2 * w2_K && w2_N == w13_K, "W8A8 expert dimensions mismatch");
  const int64_t tokens = input.size(0), top_k = topk_ids.size(1), experts = w13_packed.size(0);

  fmoe_workspace_layout layout;
  TORCH_CHECK(fmoe_w8a8_workspace_layout(tokens, static_cast<int>(top_k), static_cast<int>(experts), static_cast<int>(w13_K),
                                         static_cast<int>(w2_K), &layout) == FMOE_OK,
              fmoe_last_error());
  // The reference keeps these buffers in a thread-local scratch; a caching allocator plays that role here.
  at::Tensor workspace = at::empty({static_cast<int64_t>(layout.total_bytes) + 256}, input.options().dtype(at::kByte));
  void* aligned = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(workspace.data_ptr()) + 255) & ~static_cast<uintptr_t>(255));
  at::Tensor result = out.has_value() ? *out : at::empty_like(input);

  fmoe_config config = {};
  config.swiglu_limit = static_cast<float>(swiglu_limit);
  config.gate_up_tile = first_or_zero(task_w13_window_tiles);
  config.down_tile = first_or_zero(task_w2_window_tiles);
  const int status = fmoe_w8a8_forward(
      input.data_ptr(), w13_packed.data_ptr<int8_t>(), w13_scales.data_ptr<float>(), w2_packed.data_ptr<int8_t>(),
      w2_scales.data_ptr<float>(), topk_weights.data_ptr<float>(), topk_ids.data_ptr<int64_t>(), tokens, static_cast<int>(top_k),
      static_cast<int>(experts), static_cast<int>(w13_K), static_cast<int>(w2_K), &config, result.data_ptr(), aligned,
      layout.total_bytes, c10::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(status == FMOE_OK, fmoe_last_error());
  // Device-detected errors (an expert id outside [0, E)) are read back like the reference's range check raises.
  int32_t error = 0, detail = 0;
  TORCH_CHECK(fmoe_read_status(aligned, c10::cuda::getCurrentCUDAStream().stream(), &error, &detail) == FMOE_OK, fmoe_last_error());
  TORCH_CHECK(error == FMOE_OK, fmoe_last_error());
  return result;
}
