// Top-k merge: out[t,:] = bf16( sum over slots of route_out[t*K+slot,:] * w[t,slot] ) in the
// reference's fixed orders, so the result is deterministic and independent of the launch shape.
//   W8A8: one fused multiply-add chain in slot order starting from zero
//         (csrc/moe/arm/i8mm_w8a8/kernels.cpp:675-688).
//   BF16: for K in {2,4,6,8} a pairwise tree over unfused products, split at the largest power of two
//         below the count; any other K the same chain as W8A8 (csrc/moe/arm/sve_bf16/route_merge.cpp:48-86).
// route_out rows are indexed by flat route id, so the un-permute already happened in the down GEMM's
// epilogue; this pass is a pure streaming read of fp32 rows with 16-byte loads.
#include "common.cuh"
#include "kernels.h"

namespace fmoe {

namespace {

constexpr int kMergeThreads = 256;
constexpr int kMaxTopK = 32;

template <int Begin, int Count>
__device__ __forceinline__ float tree_sum(const float* products) {
  if constexpr (Count == 1) {
    return products[Begin];
  } else {
    constexpr int kLeft = Count > 4 ? 4 : (Count > 2 ? 2 : 1);  // largest power of two below Count (Count <= 8)
    return __fadd_rn(tree_sum<Begin, kLeft>(products), tree_sum<Begin + kLeft, Count - kLeft>(products));
  }
}

template <int TopK>
__device__ __forceinline__ float merge_fixed(const float* values, const float* weights) {
  float products[TopK];
#pragma unroll
  for (int slot = 0; slot < TopK; ++slot) products[slot] = __fmul_rn(values[slot], weights[slot]);
  return tree_sum<0, TopK>(products);
}

// Four consecutive values of a route row as fp32.  kBf16Rows: the rows were stored as bf16 (the opt-in compact
// return of the expert-parallel path); widening is exact, the rounding happened at the store.
template <bool kBf16Rows>
__device__ __forceinline__ float4 load_row4(const void* route_out, int64_t element) {
  if constexpr (kBf16Rows) {
    const uint2 packed = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(route_out) + element);
    return make_float4(__uint_as_float(packed.x << 16), __uint_as_float(packed.x & 0xffff0000u), __uint_as_float(packed.y << 16),
                       __uint_as_float(packed.y & 0xffff0000u));
  } else {
    return *reinterpret_cast<const float4*>(static_cast<const float*>(route_out) + element);
  }
}

// Tree merge of four channels with the slot count known at compile time: every row load and every product sits in a
// register (a loop over a run-time slot count indexes its row array dynamically, which sends it to local memory).
template <int TopK, bool kBf16Rows>
__device__ __forceinline__ void tree_merge4(const void* route_out, int64_t base, int hidden, const bool* present, const float* weights,
                                            float* result) {
  float4 rows[TopK];
#pragma unroll
  for (int slot = 0; slot < TopK; ++slot) {
    rows[slot] = present[slot] ? load_row4<kBf16Rows>(route_out, base + static_cast<int64_t>(slot) * hidden) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
#pragma unroll
  for (int lane = 0; lane < 4; ++lane) {
    float values[TopK];
#pragma unroll
    for (int slot = 0; slot < TopK; ++slot) values[slot] = reinterpret_cast<const float*>(&rows[slot])[lane];
    result[lane] = merge_fixed<TopK>(values, weights);
  }
}

// Chain merge (fused multiply-adds in slot order from zero) of four channels with the slot count known at compile
// time: the row loads are issued together instead of one per loop iteration.  Same operations in the same order as
// the run-time loop.
template <int TopK, bool kBf16Rows>
__device__ __forceinline__ void chain_merge4(const void* route_out, int64_t base, int hidden, const bool* present, const float* weights,
                                             float* result) {
  float4 rows[TopK];
#pragma unroll
  for (int slot = 0; slot < TopK; ++slot) {
    rows[slot] = present[slot] ? load_row4<kBf16Rows>(route_out, base + static_cast<int64_t>(slot) * hidden) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
  result[0] = result[1] = result[2] = result[3] = 0.0f;
#pragma unroll
  for (int slot = 0; slot < TopK; ++slot) {
    const float w = weights[slot];
    result[0] = __fmaf_rn(rows[slot].x, w, result[0]);
    result[1] = __fmaf_rn(rows[slot].y, w, result[1]);
    result[2] = __fmaf_rn(rows[slot].z, w, result[2]);
    result[3] = __fmaf_rn(rows[slot].w, w, result[3]);
  }
}

// The same for eight channels of bf16 rows (one 16-byte load per slot).
template <int TopK>
__device__ __forceinline__ void tree_merge8_bf16(const uint16_t* route_out, int64_t base, int hidden, const bool* present, const float* weights,
                                                 float* result) {
  uint4 rows[TopK];
#pragma unroll
  for (int slot = 0; slot < TopK; ++slot) {
    rows[slot] = present[slot] ? *reinterpret_cast<const uint4*>(route_out + base + static_cast<int64_t>(slot) * hidden) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int lane = 0; lane < 8; ++lane) {
    float values[TopK];
#pragma unroll
    for (int slot = 0; slot < TopK; ++slot) {
      const uint32_t word = reinterpret_cast<const uint32_t*>(&rows[slot])[lane >> 1];
      values[slot] = __uint_as_float((lane & 1) ? (word & 0xffff0000u) : (word << 16));
    }
    result[lane] = merge_fixed<TopK>(values, weights);
  }
}

// The same merge over bf16 rows with eight channels per thread: one 16-byte load per slot, one 16-byte store.
__global__ void __launch_bounds__(kMergeThreads)
merge_bf16_rows8_kernel(const uint16_t* __restrict__ route_out, const float* __restrict__ topk_weights, const int* __restrict__ route_pos,
                        int top_k, int hidden, int tree, uint16_t* __restrict__ out) {
  __shared__ float weights[kMaxTopK];
  __shared__ bool present[kMaxTopK];
  const int64_t token = blockIdx.x;
  if (threadIdx.x < top_k) {
    weights[threadIdx.x] = topk_weights[token * top_k + threadIdx.x];
    present[threadIdx.x] = route_pos == nullptr || route_pos[token * top_k + threadIdx.x] >= 0;
  }
  __syncthreads();
  const int h = (blockIdx.y * kMergeThreads + threadIdx.x) * 8;
  if (h >= hidden) return;
  const int64_t base = token * top_k * static_cast<int64_t>(hidden) + h;
  const bool fixed = tree && (top_k == 2 || top_k == 4 || top_k == 6 || top_k == 8);
  float result[8];
  if (fixed) {
    switch (top_k) {
      case 2: tree_merge8_bf16<2>(route_out, base, hidden, present, weights, result); break;
      case 4: tree_merge8_bf16<4>(route_out, base, hidden, present, weights, result); break;
      case 6: tree_merge8_bf16<6>(route_out, base, hidden, present, weights, result); break;
      default: tree_merge8_bf16<8>(route_out, base, hidden, present, weights, result); break;
    }
  } else {
#pragma unroll
    for (int lane = 0; lane < 8; ++lane) result[lane] = 0.0f;
    for (int slot = 0; slot < top_k; ++slot) {
      const uint4 row = present[slot] ? *reinterpret_cast<const uint4*>(route_out + base + static_cast<int64_t>(slot) * hidden) : make_uint4(0, 0, 0, 0);
      const float w = weights[slot];
      const uint32_t words[4] = {row.x, row.y, row.z, row.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        result[2 * i] = __fmaf_rn(__uint_as_float(words[i] << 16), w, result[2 * i]);
        result[2 * i + 1] = __fmaf_rn(__uint_as_float(words[i] & 0xffff0000u), w, result[2 * i + 1]);
      }
    }
  }
  uint4 packed;
  packed.x = static_cast<uint32_t>(f32_to_bf16_bits(result[0])) | (static_cast<uint32_t>(f32_to_bf16_bits(result[1])) << 16);
  packed.y = static_cast<uint32_t>(f32_to_bf16_bits(result[2])) | (static_cast<uint32_t>(f32_to_bf16_bits(result[3])) << 16);
  packed.z = static_cast<uint32_t>(f32_to_bf16_bits(result[4])) | (static_cast<uint32_t>(f32_to_bf16_bits(result[5])) << 16);
  packed.w = static_cast<uint32_t>(f32_to_bf16_bits(result[6])) | (static_cast<uint32_t>(f32_to_bf16_bits(result[7])) << 16);
  *reinterpret_cast<uint4*>(out + token * hidden + h) = packed;
}

template <bool kBf16Rows>
__global__ void __launch_bounds__(kMergeThreads)
merge_kernel(const void* __restrict__ route_out, const float* __restrict__ topk_weights, const int* __restrict__ route_pos, int top_k,
             int hidden, int tree, uint16_t* __restrict__ out) {
  __shared__ float weights[kMaxTopK];
  __shared__ bool present[kMaxTopK];
  // Tokens ride on grid.x (up to 2^31 - 1 blocks), the few chunks of a row on grid.y (at most 65535).
  const int64_t token = blockIdx.x;
  if (threadIdx.x < top_k) {
    weights[threadIdx.x] = topk_weights[token * top_k + threadIdx.x];
    // A route dropped by the route build (expert id out of range; reported in the status block) has no row: the
    // down GEMM never wrote it, so it counts as a row of zeros instead of whatever the workspace held.
    present[threadIdx.x] = route_pos == nullptr || route_pos[token * top_k + threadIdx.x] >= 0;
  }
  __syncthreads();
  const int h = (blockIdx.y * kMergeThreads + threadIdx.x) * 4;
  if (h >= hidden) return;
  const int64_t base = token * top_k * static_cast<int64_t>(hidden) + h;
  float result[4];
  const bool fixed = tree && (top_k == 2 || top_k == 4 || top_k == 6 || top_k == 8);
  if (fixed) {
    switch (top_k) {
      case 2: tree_merge4<2, kBf16Rows>(route_out, base, hidden, present, weights, result); break;
      case 4: tree_merge4<4, kBf16Rows>(route_out, base, hidden, present, weights, result); break;
      case 6: tree_merge4<6, kBf16Rows>(route_out, base, hidden, present, weights, result); break;
      default: tree_merge4<8, kBf16Rows>(route_out, base, hidden, present, weights, result); break;
    }
  } else if (top_k == 8) {
    chain_merge4<8, kBf16Rows>(route_out, base, hidden, present, weights, result);
  } else if (top_k == 9) {
    chain_merge4<9, kBf16Rows>(route_out, base, hidden, present, weights, result);
  } else if (top_k == 4) {
    chain_merge4<4, kBf16Rows>(route_out, base, hidden, present, weights, result);
  } else {
    result[0] = result[1] = result[2] = result[3] = 0.0f;
    for (int slot = 0; slot < top_k; ++slot) {
      const float4 row = present[slot] ? load_row4<kBf16Rows>(route_out, base + static_cast<int64_t>(slot) * hidden)
                                       : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      const float w = weights[slot];
      result[0] = __fmaf_rn(row.x, w, result[0]);
      result[1] = __fmaf_rn(row.y, w, result[1]);
      result[2] = __fmaf_rn(row.z, w, result[2]);
      result[3] = __fmaf_rn(row.w, w, result[3]);
    }
  }
  uint2 packed;
  packed.x = static_cast<uint32_t>(f32_to_bf16_bits(result[0])) | (static_cast<uint32_t>(f32_to_bf16_bits(result[1])) << 16);
  packed.y = static_cast<uint32_t>(f32_to_bf16_bits(result[2])) | (static_cast<uint32_t>(f32_to_bf16_bits(result[3])) << 16);
  *reinterpret_cast<uint2*>(out + token * hidden + h) = packed;
}

}  // namespace

cudaError_t launch_merge(const float* route_out, const float* topk_weights, int64_t tokens, int top_k, int hidden,
                         int tree, uint16_t* out, cudaStream_t stream, const int* route_pos) {
  if (tokens <= 0) return cudaSuccess;
  if (top_k > kMaxTopK) return cudaErrorInvalidValue;
  const dim3 grid(static_cast<unsigned>(tokens), (hidden / 4 + kMergeThreads - 1) / kMergeThreads);
  merge_kernel<false><<<grid, kMergeThreads, 0, stream>>>(route_out, topk_weights, route_pos, top_k, hidden, tree, out);
  return cudaGetLastError();
}

cudaError_t launch_merge_bf16_rows(const uint16_t* route_out, const float* topk_weights, int64_t tokens, int top_k, int hidden,
                                   int tree, uint16_t* out, cudaStream_t stream, const int* route_pos) {
  if (tokens <= 0) return cudaSuccess;
  if (top_k > kMaxTopK) return cudaErrorInvalidValue;
  if (hidden % 8 == 0) {
    const dim3 grid8(static_cast<unsigned>(tokens), (hidden / 8 + kMergeThreads - 1) / kMergeThreads);
    merge_bf16_rows8_kernel<<<grid8, kMergeThreads, 0, stream>>>(route_out, topk_weights, route_pos, top_k, hidden, tree, out);
    return cudaGetLastError();
  }
  const dim3 grid(static_cast<unsigned>(tokens), (hidden / 4 + kMergeThreads - 1) / kMergeThreads);
  merge_kernel<true><<<grid, kMergeThreads, 0, stream>>>(route_out, topk_weights, route_pos, top_k, hidden, tree, out);
  return cudaGetLastError();
}

}  // namespace fmoe
