// Diagnostic grouped GEMM on CUDA cores (dp4a for int8, fp32 FMA for bf16).
//
// Not the product path: it exists as a stage-level cross-check of the tcgen05 kernel, in the way the
// reference exposes single stages through its fused_moe_test_* bindings (csrc/moe/module.cpp:41-115).
// It computes the same two stages with the same epilogues:
//   gate_up: acc[r,n] = sum_k A[r,k] * W13[e,n,k]  ->  dequant, clamp, SiLU(gate)*up, bf16
//            (run_stage + w13_epilogue, csrc/moe/arm/i8mm_w8a8/kernels.cpp:328-368, 230-246)
//   down:    acc[r,h] = sum_i Y[r,i] * W2[e,h,i]   ->  route_out[flat(r), h] = f32(acc) * scales
//            (run_stage + store_w2, csrc/moe/arm/i8mm_w8a8/kernels.cpp:248-257, 659-671)
// A work item is (expert, first row, rows <= 8).  One warp owns one output channel (gate_up: the
// gate/up channel pair) and streams that weight row once with 16-byte loads while the item's
// activation rows come from L1/L2; the K reduction finishes with warp shuffles.
#include "common.cuh"
#include "kernels.h"

namespace fmoe {

namespace {

constexpr int kSimtWarps = 8;

__device__ __forceinline__ int dp4a_u4(const uint4& a, const uint4& b, int acc) {
  acc = __dp4a(static_cast<int>(a.x), static_cast<int>(b.x), acc);
  acc = __dp4a(static_cast<int>(a.y), static_cast<int>(b.y), acc);
  acc = __dp4a(static_cast<int>(a.z), static_cast<int>(b.z), acc);
  acc = __dp4a(static_cast<int>(a.w), static_cast<int>(b.w), acc);
  return acc;
}

__device__ __forceinline__ float dot8_bf16(const uint4& a, const uint4& b, float acc) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
  const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc = __fmaf_rn(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), acc);
    acc = __fmaf_rn(__uint_as_float(aw[i] & 0xffff0000u), __uint_as_float(bw[i] & 0xffff0000u), acc);
  }
  return acc;
}

template <bool kInt8, bool kGateUp>
__global__ void __launch_bounds__(kSimtWarps * 32)
simt_grouped_gemm_kernel(GroupedGemmArgs args) {
  using Acc = typename std::conditional<kInt8, int, float>::type;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int items = min(args.status[args.item_count_word], args.max_items);
  const int elem_bytes = kInt8 ? 1 : 2;
  const int vecs = (args.k * elem_bytes) >> 4;  // 16-byte vectors per row
  const int n_total = kGateUp ? 2 * args.n_out : args.n_out;
  const char* a_base = static_cast<const char*>(args.a_rows);
  const char* w_base = static_cast<const char*>(args.weights);
  const int64_t row_bytes = static_cast<int64_t>(args.k) * elem_bytes;

  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int expert = args.items[4 * item + 0];
    const int row0 = args.items[4 * item + 1];
    const int rows = args.items[4 * item + 2];
    const char* w_expert = w_base + static_cast<int64_t>(expert) * n_total * row_bytes;
    for (int n = blockIdx.y * kSimtWarps + warp; n < args.n_out; n += gridDim.y * kSimtWarps) {
      Acc acc0[kSimtRowTile];
      Acc acc1[kSimtRowTile];
#pragma unroll
      for (int r = 0; r < kSimtRowTile; ++r) {
        acc0[r] = 0;
        acc1[r] = 0;
      }
      const uint4* w0 = reinterpret_cast<const uint4*>(w_expert + static_cast<int64_t>(n) * row_bytes);
      const uint4* w1 = reinterpret_cast<const uint4*>(w_expert + static_cast<int64_t>(n + args.n_out) * row_bytes);
      for (int v = lane; v < vecs; v += 32) {
        const uint4 wv0 = w0[v];
        uint4 wv1 = wv0;
        if (kGateUp) wv1 = w1[v];
#pragma unroll
        for (int r = 0; r < kSimtRowTile; ++r) {
          if (r < rows) {
            const uint4 av = *reinterpret_cast<const uint4*>(a_base + static_cast<int64_t>(row0 + r) * row_bytes + 16 * static_cast<int64_t>(v));
            if constexpr (kInt8) {
              acc0[r] = dp4a_u4(av, wv0, acc0[r]);
              if (kGateUp) acc1[r] = dp4a_u4(av, wv1, acc1[r]);
            } else {
              acc0[r] = dot8_bf16(av, wv0, acc0[r]);
              if (kGateUp) acc1[r] = dot8_bf16(av, wv1, acc1[r]);
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < kSimtRowTile; ++r) {
        acc0[r] = warp_sum(acc0[r]);
        if (kGateUp) acc1[r] = warp_sum(acc1[r]);
      }
      // Lane r finishes row r.
      Acc mine0 = 0, mine1 = 0;
#pragma unroll
      for (int r = 0; r < kSimtRowTile; ++r) {
        if (lane == r) {
          mine0 = acc0[r];
          mine1 = acc1[r];
        }
      }
      if (lane < rows) {
        const int64_t row = row0 + lane;
        if (args.dump_acc) {
          Acc* dump = static_cast<Acc*>(args.dump_acc) + row * n_total;
          dump[n] = mine0;
          if (kGateUp) dump[n + args.n_out] = mine1;
        }
        if constexpr (kGateUp) {
          float gate, up;
          if constexpr (kInt8) {
            const float a = args.a_scale[row];
            const float* s = args.w_scale + static_cast<int64_t>(expert) * n_total;
            gate = dequantize(mine0, a, s[n], args.numerics);
            up = dequantize(mine1, a, s[n + args.n_out], args.numerics);
          } else {
            gate = mine0;
            up = mine1;
          }
          args.y[row * args.n_out + n] = swiglu_to_bf16(gate, up, args.swiglu_limit);
        } else {
          float value;
          if constexpr (kInt8) {
            value = dequantize(mine0, args.a_scale[row], args.w_scale[static_cast<int64_t>(expert) * n_total + n], args.numerics);
          } else {
            value = mine0;
          }
          if (args.dense_out != nullptr) {
            if (args.bias != nullptr) value = __fadd_rn(value, args.bias[n]);
            if (args.dense_out_bf16) {
              static_cast<uint16_t*>(args.dense_out)[row * args.n_out + n] = f32_to_bf16_bits(value);
            } else {
              static_cast<float*>(args.dense_out)[row * args.n_out + n] = value;
            }
          } else {
            const int64_t flat = args.sorted_routes[row];
            args.route_out[flat * args.n_out + n] = value;
          }
        }
      }
    }
  }
}

}  // namespace

cudaError_t launch_simt_grouped_gemm(const GroupedGemmArgs& args, bool int8, bool gate_up, cudaStream_t stream) {
  if (args.max_items <= 0 || args.total_rows <= 0) return cudaSuccess;
  const int grid_x = args.max_items < 4096 ? args.max_items : 4096;
  int grid_y = (args.n_out + kSimtWarps - 1) / kSimtWarps;
  if (grid_y > 32) grid_y = 32;
  const dim3 grid(grid_x, grid_y);
  const dim3 block(kSimtWarps * 32);
  if (int8 && gate_up) simt_grouped_gemm_kernel<true, true><<<grid, block, 0, stream>>>(args);
  if (int8 && !gate_up) simt_grouped_gemm_kernel<true, false><<<grid, block, 0, stream>>>(args);
  if (!int8 && gate_up) simt_grouped_gemm_kernel<false, true><<<grid, block, 0, stream>>>(args);
  if (!int8 && !gate_up) simt_grouped_gemm_kernel<false, false><<<grid, block, 0, stream>>>(args);
  return cudaGetLastError();
}

}  // namespace fmoe
