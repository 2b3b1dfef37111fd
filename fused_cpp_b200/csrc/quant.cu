// Dynamic per-row symmetric int8 quantisation and the row gather of the BF16 path.
//
// The reference quantises x[token] once per route into the expert's private buffer
// (quantize_bf16_row, csrc/moe/arm/i8mm_w8a8/kernels.cpp:211-228, called at :639-644 and :655-656).
// One CTA handles one output row: pass 1 finds the row's absmax with 16-byte loads and a
// warp-shuffle/shared-memory reduction, pass 2 re-reads the row (L1/L2 resident) and stores 16 int8
// per thread as one 16-byte vector.  With `sorted_routes` the source row is the route's token, so
// the output is already in expert-sorted order for the grouped GEMM (gather and quantise fused).
#include "common.cuh"
#include "kernels.h"

namespace fmoe {

namespace {

constexpr int kQuantThreads = 256;

__device__ __forceinline__ float block_max(float value, float* smem) {
  value = warp_max(value);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = value;
  __syncthreads();
  float result = lane < (blockDim.x >> 5) ? smem[lane] : 0.0f;
  result = warp_max(result);
  __syncthreads();
  return result;
}

__device__ __forceinline__ void unpack8(const uint4& v, float* out) {
  const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(words[i] << 16);
    out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ float amax8(const uint4& v) {
  float values[8];
  unpack8(v, values);
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(values[i]));
  return m;
}

// operand: 1/scale (NATIVE) or scale (TORCHREF); inverse: 1/scale, used by the TORCHREF fast path.
__device__ __forceinline__ uint32_t pack4(const float* values, float operand, float inverse, int numerics) {
  if (numerics == FMOE_NUMERICS_TORCHREF) return quantize4_torchref_fast(values, operand, inverse);
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    packed |= (static_cast<uint32_t>(quantize_value(values[i], operand, numerics)) & 0xffu) << (8 * i);
  }
  return packed;
}

// cols % 16 == 0.  One CTA per output row.
__global__ void __launch_bounds__(kQuantThreads)
quantize_rows_kernel(const uint16_t* __restrict__ x, int cols, const int* __restrict__ sorted_routes, int top_k,
                     const int* __restrict__ valid_rows, int numerics, int weight_mode, int8_t* __restrict__ q,
                     float* __restrict__ scale_out) {
  __shared__ float smem[32];
  const int64_t row = blockIdx.x;
  if (valid_rows && row >= *valid_rows) return;  // rows of dropped (out-of-range) routes
  const int64_t src_row = sorted_routes ? static_cast<int64_t>(sorted_routes[row] / top_k) : row;
  const uint4* src = reinterpret_cast<const uint4*>(x + src_row * cols);
  const int vec16 = cols >> 4;
  float local = 0.0f;
  for (int v = threadIdx.x; v < vec16; v += kQuantThreads) {
    local = fmaxf(local, amax8(src[2 * v]));
    local = fmaxf(local, amax8(src[2 * v + 1]));
  }
  const float amax = block_max(local, smem);
  float scale;
  int mode = numerics;
  if (weight_mode) {
    scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    mode = FMOE_NUMERICS_TORCHREF;
  } else {
    scale = row_scale_from_amax(amax, numerics);
  }
  if (threadIdx.x == 0) scale_out[row] = scale;
  const float operand = quantize_operand(scale, mode);
  const float inverse = __fdiv_rn(1.0f, scale);
  uint4* dst = reinterpret_cast<uint4*>(q + row * cols);
  for (int v = threadIdx.x; v < vec16; v += kQuantThreads) {
    float values[16];
    unpack8(src[2 * v], values);
    unpack8(src[2 * v + 1], values + 8);
    uint4 out;
    out.x = pack4(values, operand, inverse, mode);
    out.y = pack4(values + 4, operand, inverse, mode);
    out.z = pack4(values + 8, operand, inverse, mode);
    out.w = pack4(values + 12, operand, inverse, mode);
    dst[v] = out;
  }
}

// Same work, one warp per output row, for rows of at most 32 * 16 * kVectors columns: the row is read once
// into registers (kVectors 32-byte pieces per lane), the absmax is a shuffle reduction, no block barrier.
// Rows of a few KB (the 2048-column intermediate of the W8A8 layer) are too short to keep a 256-thread CTA busy.
template <int kVectors>
__global__ void __launch_bounds__(kQuantThreads)
quantize_rows_warp_kernel(const uint16_t* __restrict__ x, int64_t out_rows, int cols, const int* __restrict__ sorted_routes, int top_k,
                          const int* __restrict__ valid_rows, int numerics, int weight_mode, int8_t* __restrict__ q,
                          float* __restrict__ scale_out) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kQuantThreads / 32) + (threadIdx.x >> 5);
  if (row >= out_rows) return;
  if (valid_rows && row >= *valid_rows) return;
  const int64_t src_row = sorted_routes ? static_cast<int64_t>(sorted_routes[row] / top_k) : row;
  const uint4* src = reinterpret_cast<const uint4*>(x + src_row * cols);
  const int vec16 = cols >> 4;
  uint4 held[kVectors][2];
  float local = 0.0f;
#pragma unroll
  for (int i = 0; i < kVectors; ++i) {
    const int v = lane + 32 * i;
    if (v < vec16) {
      held[i][0] = src[2 * v];
      held[i][1] = src[2 * v + 1];
      local = fmaxf(local, fmaxf(amax8(held[i][0]), amax8(held[i][1])));
    }
  }
  const float amax = warp_max(local);
  float scale;
  int mode = numerics;
  if (weight_mode) {
    scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    mode = FMOE_NUMERICS_TORCHREF;
  } else {
    scale = row_scale_from_amax(amax, numerics);
  }
  if (lane == 0) scale_out[row] = scale;
  const float operand = quantize_operand(scale, mode);
  const float inverse = __fdiv_rn(1.0f, scale);
  uint4* dst = reinterpret_cast<uint4*>(q + row * cols);
#pragma unroll
  for (int i = 0; i < kVectors; ++i) {
    const int v = lane + 32 * i;
    if (v < vec16) {
      float values[16];
      unpack8(held[i][0], values);
      unpack8(held[i][1], values + 8);
      uint4 out;
      out.x = pack4(values, operand, inverse, mode);
      out.y = pack4(values + 4, operand, inverse, mode);
      out.z = pack4(values + 8, operand, inverse, mode);
      out.w = pack4(values + 12, operand, inverse, mode);
      dst[v] = out;
    }
  }
}

// cols % 16 == 0, top_k <= 32.  One CTA per token: the row is quantised once and stored to each of its routes'
// sorted positions (the reference re-quantises the token for every route, kernels.cpp:639-644; the bits are the same).
__global__ void __launch_bounds__(kQuantThreads)
quantize_tokens_scatter_kernel(const uint16_t* __restrict__ x, int cols, int top_k, const int* __restrict__ route_pos,
                               int numerics, int8_t* __restrict__ q, float* __restrict__ scale_out) {
  __shared__ float smem[32];
  __shared__ int positions[32];
  const int64_t token = blockIdx.x;
  if (threadIdx.x < top_k) positions[threadIdx.x] = route_pos[token * top_k + threadIdx.x];
  const uint4* src = reinterpret_cast<const uint4*>(x + token * cols);
  const int vec16 = cols >> 4;
  float local = 0.0f;
  for (int v = threadIdx.x; v < vec16; v += kQuantThreads) {
    local = fmaxf(local, amax8(src[2 * v]));
    local = fmaxf(local, amax8(src[2 * v + 1]));
  }
  const float amax = block_max(local, smem);  // its barriers also publish positions[]
  const float scale = row_scale_from_amax(amax, numerics);
  if (threadIdx.x < top_k && positions[threadIdx.x] >= 0) scale_out[positions[threadIdx.x]] = scale;
  const float operand = quantize_operand(scale, numerics);
  const float inverse = __fdiv_rn(1.0f, scale);
  for (int v = threadIdx.x; v < vec16; v += kQuantThreads) {
    float values[16];
    unpack8(src[2 * v], values);
    unpack8(src[2 * v + 1], values + 8);
    uint4 out;
    out.x = pack4(values, operand, inverse, numerics);
    out.y = pack4(values + 4, operand, inverse, numerics);
    out.z = pack4(values + 8, operand, inverse, numerics);
    out.w = pack4(values + 12, operand, inverse, numerics);
    for (int slot = 0; slot < top_k; ++slot) {
      const int position = positions[slot];
      if (position >= 0) reinterpret_cast<uint4*>(q + static_cast<int64_t>(position) * cols)[v] = out;
    }
  }
}

// W8A16 in its fixed-point form.  cols % 16 == 0.  One CTA per route row p (gathered by token when sorted_routes is
// given): the bf16 row becomes 16-bit fixed point (plane_fixed_point) and is stored as two int8 rows, the high plane at
// row 2p and the low plane at row 2p + 1 of `planes`; scale_out[p] is the row scale.
__global__ void __launch_bounds__(kQuantThreads)
split_rows_planes_kernel(const uint16_t* __restrict__ x, int cols, const int* __restrict__ sorted_routes, int top_k,
                         const int* __restrict__ valid_rows, int8_t* __restrict__ planes, float* __restrict__ scale_out) {
  __shared__ float smem[32];
  const int64_t row = blockIdx.x;
  if (valid_rows && row >= *valid_rows) return;
  const int64_t src_row = sorted_routes ? static_cast<int64_t>(sorted_routes[row] / top_k) : row;
  const uint4* src = reinterpret_cast<const uint4*>(x + src_row * cols);
  const int vec16 = cols >> 4;
  float local = 0.0f;
  for (int v = threadIdx.x; v < vec16; v += kQuantThreads) {
    local = fmaxf(local, amax8(src[2 * v]));
    local = fmaxf(local, amax8(src[2 * v + 1]));
  }
  const float amax = block_max(local, smem);
  const float scale = plane_row_scale(amax);
  if (threadIdx.x == 0) scale_out[row] = scale;
  uint4* high_row = reinterpret_cast<uint4*>(planes + (2 * row) * cols);
  uint4* low_row = reinterpret_cast<uint4*>(planes + (2 * row + 1) * cols);
  for (int v = threadIdx.x; v < vec16; v += kQuantThreads) {
    float values[16];
    unpack8(src[2 * v], values);
    unpack8(src[2 * v + 1], values + 8);
    uint32_t high[4] = {0, 0, 0, 0};
    uint32_t low[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int fixed = plane_fixed_point(values[i], scale);
      const int low_part = ((fixed + 128) & 255) - 128;
      const int high_part = (fixed - low_part) >> 8;  // fixed - low_part is a multiple of 256
      high[i >> 2] |= (static_cast<uint32_t>(high_part) & 0xffu) << (8 * (i & 3));
      low[i >> 2] |= (static_cast<uint32_t>(low_part) & 0xffu) << (8 * (i & 3));
    }
    high_row[v] = make_uint4(high[0], high[1], high[2], high[3]);
    low_row[v] = make_uint4(low[0], low[1], low[2], low[3]);
  }
}

// The same split once per TOKEN, stored to the sorted positions of its top_k routes (route_pos, -1 = dropped): the bits
// every route would get from split_rows_planes_kernel, one read of x and one fixed-point conversion per token.
__global__ void __launch_bounds__(kQuantThreads)
split_tokens_scatter_planes_kernel(const uint16_t* __restrict__ x, int cols, int top_k, const int* __restrict__ route_pos,
                                   int8_t* __restrict__ planes, float* __restrict__ scale_out) {
  __shared__ float smem[32];
  __shared__ int positions[32];
  const int64_t token = blockIdx.x;
  if (threadIdx.x < top_k) positions[threadIdx.x] = route_pos[token * top_k + threadIdx.x];
  const uint4* src = reinterpret_cast<const uint4*>(x + token * cols);
  const int vec16 = cols >> 4;
  float local = 0.0f;
  for (int v = threadIdx.x; v < vec16; v += kQuantThreads) {
    local = fmaxf(local, amax8(src[2 * v]));
    local = fmaxf(local, amax8(src[2 * v + 1]));
  }
  const float amax = block_max(local, smem);  // its barriers also publish positions[]
  const float scale = plane_row_scale(amax);
  if (threadIdx.x < top_k && positions[threadIdx.x] >= 0) scale_out[positions[threadIdx.x]] = scale;
  for (int v = threadIdx.x; v < vec16; v += kQuantThreads) {
    float values[16];
    unpack8(src[2 * v], values);
    unpack8(src[2 * v + 1], values + 8);
    uint32_t high[4] = {0, 0, 0, 0};
    uint32_t low[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int fixed = plane_fixed_point(values[i], scale);
      const int low_part = ((fixed + 128) & 255) - 128;
      const int high_part = (fixed - low_part) >> 8;
      high[i >> 2] |= (static_cast<uint32_t>(high_part) & 0xffu) << (8 * (i & 3));
      low[i >> 2] |= (static_cast<uint32_t>(low_part) & 0xffu) << (8 * (i & 3));
    }
    const uint4 high_vector = make_uint4(high[0], high[1], high[2], high[3]);
    const uint4 low_vector = make_uint4(low[0], low[1], low[2], low[3]);
    for (int slot = 0; slot < top_k; ++slot) {
      const int64_t position = positions[slot];
      if (position >= 0) {
        reinterpret_cast<uint4*>(planes + (2 * position) * cols)[v] = high_vector;
        reinterpret_cast<uint4*>(planes + (2 * position + 1) * cols)[v] = low_vector;
      }
    }
  }
}

// Dense linear: arbitrary cols, fp32 or bf16 source, zero-padded to cols_padded, clamp to [-128,127]
// (single GEMM) or [-127,127] (paired GEMMs) with division and ties-to-even (csrc/i8gemm.cpp:384-399, :492-506).
// Status block and work items of the dense GEMM that follows (one "expert", row tiles of row_tile rows; the group key
// of decode_unit in the fourth word), written by block 0 of the quantiser so that the op needs no launches of its own
// for them.  Every status word is written: the block starts out in an unknown state.
struct DenseItems {
  int64_t rows;
  int row_tile;
  int max_items;
  int* items;
  int* status;
};

__device__ __forceinline__ void write_dense_items(const DenseItems& d) {
  const int tiles = static_cast<int>((d.rows + d.row_tile - 1) / d.row_tile);
  const int count = tiles < d.max_items ? tiles : d.max_items;
  for (int t = threadIdx.x; t < count; t += blockDim.x) {
    d.items[4 * t + 0] = 0;
    d.items[4 * t + 1] = t * d.row_tile;
    d.items[4 * t + 2] = static_cast<int>(min(static_cast<int64_t>(d.row_tile), d.rows - static_cast<int64_t>(t) * d.row_tile));
    d.items[4 * t + 3] = count < 2048 ? (0 | (count << 20)) : (t | (1 << 20));
  }
  if (threadIdx.x < kStatusWords) {
    const int word = threadIdx.x;
    d.status[word] = (word == kStatusItems || word == kStatusItemsB) ? count : word == kStatusActive ? (d.rows > 0 ? 1 : 0) : 0;
  }
}

__global__ void __launch_bounds__(kQuantThreads)
quantize_rows_dense_kernel(const void* __restrict__ x, int x_is_bf16, int cols, int cols_padded, float clamp_low,
                           int8_t* __restrict__ q, float* __restrict__ scale_out, DenseItems dense_items) {
  if (blockIdx.x == 0) write_dense_items(dense_items);
  __shared__ float smem[32];
  const int64_t row = blockIdx.x;
  const float* xf = static_cast<const float*>(x) + row * cols;
  const uint16_t* xb = static_cast<const uint16_t*>(x) + row * cols;
  float local = 0.0f;
  for (int c = threadIdx.x; c < cols; c += kQuantThreads) {
    const float value = x_is_bf16 ? bf16_bits_to_f32(xb[c]) : xf[c];
    local = fmaxf(local, fabsf(value));
  }
  const float amax = block_max(local, smem);
  const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  if (threadIdx.x == 0) scale_out[row] = scale;
  int8_t* dst = q + row * cols_padded;
  for (int c = threadIdx.x; c < cols_padded; c += kQuantThreads) {
    int value = 0;
    if (c < cols) {
      const float source = x_is_bf16 ? bf16_bits_to_f32(xb[c]) : xf[c];
      float rounded = rintf(__fdiv_rn(source, scale));
      rounded = fmaxf(fminf(rounded, 127.0f), clamp_low);
      value = static_cast<int>(rounded);
    }
    dst[c] = static_cast<int8_t>(value);
  }
}

// cols % 8 == 0.  out[p] = x[sorted_routes[p] / top_k].
__global__ void __launch_bounds__(kQuantThreads)
gather_rows_kernel(const uint16_t* __restrict__ x, int cols, const int* __restrict__ sorted_routes, int top_k,
                   const int* __restrict__ valid_rows, uint16_t* __restrict__ out) {
  const int64_t row = blockIdx.x;
  if (valid_rows && row >= *valid_rows) return;
  const int64_t src_row = sorted_routes[row] / top_k;
  const uint4* src = reinterpret_cast<const uint4*>(x + src_row * cols);
  uint4* dst = reinterpret_cast<uint4*>(out + row * cols);
  for (int v = threadIdx.x; v < (cols >> 3); v += kQuantThreads) dst[v] = src[v];
}

__global__ void gather_scalars_kernel(const float* __restrict__ in, int64_t n, const int* __restrict__ index,
                                      const int* __restrict__ valid_rows, float* __restrict__ out) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= n || (valid_rows && i >= *valid_rows)) return;
  out[i] = in[index[i]];
}

}  // namespace

cudaError_t launch_gather_scalars(const float* in, int64_t n, const int* index, const int* valid_rows, float* out,
                                  cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  gather_scalars_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(in, n, index, valid_rows, out);
  return cudaGetLastError();
}

cudaError_t launch_quantize_rows(const uint16_t* x, int64_t out_rows, int cols, const int* sorted_routes, int top_k,
                                 const int* valid_rows, int numerics, int weight_mode, int8_t* q, float* scale,
                                 cudaStream_t stream) {
  if (out_rows <= 0) return cudaSuccess;
  const int vec16 = cols >> 4;
  const unsigned warp_blocks = static_cast<unsigned>((out_rows + kQuantThreads / 32 - 1) / (kQuantThreads / 32));
  // A few rows (decode): one CTA per row spreads a row over 256 threads, where one warp per row would walk its 64
  // values per lane alone on an SM (10.7 us against the other kernel's ~5 us for 8 rows of 2048 columns).
  const bool few_rows = out_rows <= 592;  // four CTAs per SM at most
  if (few_rows) {
    quantize_rows_kernel<<<static_cast<unsigned>(out_rows), kQuantThreads, 0, stream>>>(x, cols, sorted_routes, top_k, valid_rows,
                                                                                       numerics, weight_mode, q, scale);
    return cudaGetLastError();
  }
  if (vec16 <= 64) {
    quantize_rows_warp_kernel<2><<<warp_blocks, kQuantThreads, 0, stream>>>(x, out_rows, cols, sorted_routes, top_k, valid_rows, numerics,
                                                                             weight_mode, q, scale);
  } else if (vec16 <= 128) {
    quantize_rows_warp_kernel<4><<<warp_blocks, kQuantThreads, 0, stream>>>(x, out_rows, cols, sorted_routes, top_k, valid_rows, numerics,
                                                                             weight_mode, q, scale);
  } else {
    quantize_rows_kernel<<<static_cast<unsigned>(out_rows), kQuantThreads, 0, stream>>>(x, cols, sorted_routes, top_k, valid_rows,
                                                                                       numerics, weight_mode, q, scale);
  }
  return cudaGetLastError();
}

cudaError_t launch_split_rows_planes(const uint16_t* x, int64_t out_rows, int cols, const int* sorted_routes, int top_k,
                                     const int* valid_rows, int8_t* planes, float* scale, cudaStream_t stream) {
  if (out_rows <= 0) return cudaSuccess;
  split_rows_planes_kernel<<<static_cast<unsigned>(out_rows), kQuantThreads, 0, stream>>>(x, cols, sorted_routes, top_k, valid_rows, planes,
                                                                                         scale);
  return cudaGetLastError();
}

cudaError_t launch_split_tokens_scatter_planes(const uint16_t* x, int64_t tokens, int cols, int top_k, const int* route_pos, int8_t* planes,
                                               float* scale, cudaStream_t stream) {
  if (tokens <= 0) return cudaSuccess;
  split_tokens_scatter_planes_kernel<<<static_cast<unsigned>(tokens), kQuantThreads, 0, stream>>>(x, cols, top_k, route_pos, planes, scale);
  return cudaGetLastError();
}

cudaError_t launch_quantize_tokens_scatter(const uint16_t* x, int64_t tokens, int cols, int top_k, const int* route_pos,
                                           int numerics, int8_t* q, float* scale, cudaStream_t stream) {
  if (tokens <= 0) return cudaSuccess;
  quantize_tokens_scatter_kernel<<<static_cast<unsigned>(tokens), kQuantThreads, 0, stream>>>(x, cols, top_k, route_pos, numerics, q,
                                                                                             scale);
  return cudaGetLastError();
}

// The same quantiser for bf16 rows whose length is a multiple of 8: 16-byte loads, 8-byte stores, and the division
// replaced as in quantize4_torchref_fast (the statement is the same clamp(rint(x / scale)); with scale = amax / 127 of
// the same row no quotient rounds below -127, so the lower clamp of -128 some callers ask for never binds).
__global__ void __launch_bounds__(kQuantThreads)
quantize_rows_dense_bf16x8_kernel(const uint16_t* __restrict__ x, int cols, int cols_padded, int8_t* __restrict__ q,
                                  float* __restrict__ scale_out, DenseItems dense_items) {
  __shared__ float smem[32];
  if (blockIdx.x == 0) write_dense_items(dense_items);
  const int64_t row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + row * cols);
  const int vec8 = cols >> 3;
  float local = 0.0f;
  for (int v = threadIdx.x; v < vec8; v += kQuantThreads) local = fmaxf(local, amax8(src[v]));
  const float amax = block_max(local, smem);
  const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  if (threadIdx.x == 0) scale_out[row] = scale;
  const float inverse = __fdiv_rn(1.0f, scale);
  uint2* dst = reinterpret_cast<uint2*>(q + row * cols_padded);
  const int vec8_padded = cols_padded >> 3;
  for (int v = threadIdx.x; v < vec8_padded; v += kQuantThreads) {
    uint2 out = make_uint2(0u, 0u);
    if (v < vec8) {
      float values[8];
      unpack8(src[v], values);
      out.x = quantize4_torchref_fast(values, scale, inverse);
      out.y = quantize4_torchref_fast(values + 4, scale, inverse);
    }
    dst[v] = out;
  }
}

cudaError_t launch_quantize_rows_dense(const void* x, int x_is_bf16, int64_t rows, int cols, int cols_padded, int clamp_low,
                                       int8_t* q, float* scale, int row_tile, int max_items, int* items, int* status,
                                       cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  const DenseItems dense_items = {rows, row_tile, max_items, items, status};
  const bool vector_form = x_is_bf16 && cols % 8 == 0 && cols_padded % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
                           (reinterpret_cast<uintptr_t>(q) & 7u) == 0;
  if (vector_form) {
    quantize_rows_dense_bf16x8_kernel<<<static_cast<unsigned>(rows), kQuantThreads, 0, stream>>>(static_cast<const uint16_t*>(x), cols,
                                                                                                cols_padded, q, scale, dense_items);
  } else {
    quantize_rows_dense_kernel<<<static_cast<unsigned>(rows), kQuantThreads, 0, stream>>>(
        x, x_is_bf16, cols, cols_padded, static_cast<float>(clamp_low), q, scale, dense_items);
  }
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const uint16_t* x, int64_t out_rows, int cols, const int* sorted_routes, int top_k,
                               const int* valid_rows, uint16_t* out, cudaStream_t stream) {
  if (out_rows <= 0) return cudaSuccess;
  gather_rows_kernel<<<static_cast<unsigned>(out_rows), kQuantThreads, 0, stream>>>(x, cols, sorted_routes, top_k, valid_rows, out);
  return cudaGetLastError();
}

}  // namespace fmoe
