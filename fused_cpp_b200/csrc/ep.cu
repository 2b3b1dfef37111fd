// Small kernels around the expert-parallel exchange.
//
// The reference has no expert parallelism (it rejects expert id remapping,
// csrc/moe/arm/i8mm_w8a8/kernels.cpp:488), so nothing here has a counterpart; the arithmetic of every
// route is unchanged by the sharding: a route is quantised where its token lives, multiplied where its
// expert lives, and merged, in the reference's slot order, where its token lives.
#include "common.cuh"
#include "kernels.h"

namespace fmoe {

namespace {

// shared_rank >= 0: id == experts_global names the replicated shared expert, served by this rank itself.
__global__ void dest_ranks_kernel(const int64_t* __restrict__ ids, int64_t n, int experts_global, int experts_per_rank,
                                  int shared_rank, int64_t* __restrict__ dest) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const int64_t id = ids[i];
  int64_t rank = (id >= 0 && id < experts_global) ? id / experts_per_rank : -1;
  if (shared_rank >= 0 && id == experts_global) rank = shared_rank;
  dest[i] = rank;
}

__global__ void local_experts_kernel(const int64_t* __restrict__ ids, const int* __restrict__ order, int64_t n,
                                     const int* __restrict__ valid_rows, int experts_global, int experts_per_rank,
                                     int64_t* __restrict__ local) {
  const int64_t p = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (p >= n || (valid_rows && p >= *valid_rows)) return;
  const int64_t id = ids[order[p]];
  local[p] = id >= experts_global ? experts_per_rank : id % experts_per_rank;  // the shared expert follows the routed ones
}

__global__ void scatter_rows_f32_kernel(const float* __restrict__ rows, const int* __restrict__ order, const int* __restrict__ valid_rows,
                                        int hidden, float* __restrict__ route_out) {
  const int64_t p = blockIdx.x;
  if (valid_rows && p >= *valid_rows) return;
  const float4* src = reinterpret_cast<const float4*>(rows + p * hidden);
  float4* dst = reinterpret_cast<float4*>(route_out + static_cast<int64_t>(order[p]) * hidden);
  for (int v = threadIdx.x; v < (hidden >> 2); v += blockDim.x) dst[v] = src[v];
}

// ---- peer-memory path: rows go straight into the expert rank's receive slab, results straight back ----

// Barrier between the ranks of the box, through flags in the slabs.  Every rank bumps its own epoch, (optionally)
// tells every destination how many rows it has just stored there, then stores the epoch into its flag in every
// rank's slab and waits until all flags in its own slab have reached that epoch.  The stores of the kernels that
// ran before it on this stream are complete when it starts (stream order), and the fence orders its own stores,
// so a rank that sees the flag also sees the rows.  The wait is bounded: after limit_ns it records
// FMOE_ERR_DEVICE_WAIT (detail = the rank it waited for) and returns.
__global__ void __launch_bounds__(64)
peer_barrier_kernel(const uint64_t* __restrict__ peer_slabs, PeerSlabLayout slab, const int* __restrict__ dest_counts, int world, int rank,
                    unsigned* __restrict__ epoch_counter, int* status, unsigned long long limit_ns) {
  __shared__ unsigned epoch_shared;
  if (threadIdx.x == 0) {
    epoch_shared = *epoch_counter + 1u;
    *epoch_counter = epoch_shared;
  }
  __syncthreads();
  const unsigned epoch = epoch_shared;
  const int peer = threadIdx.x;
  if (peer >= world) return;
  const uint64_t theirs = peer_slabs[peer];
  if (dest_counts != nullptr) *reinterpret_cast<volatile int*>(theirs + slab.counts + sizeof(int) * rank) = dest_counts[peer];
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs + slab.flags + sizeof(unsigned) * rank), "r"(epoch) : "memory");
  const uint64_t mine = peer_slabs[rank] + slab.flags + sizeof(unsigned) * peer;
  unsigned long long start = 0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
  while (true) {
    unsigned seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (static_cast<int>(seen - epoch) >= 0) break;
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - start > limit_ns) {
      raise_error(status, FMOE_ERR_DEVICE_WAIT, peer);
      break;
    }
  }
}

__device__ __forceinline__ void unpack8_bf16(const uint4& v, float* out) {
  const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(words[i] << 16);
    out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
  }
}

// One CTA per token.  A destination's slab is divided into one region of `region` rows per source rank, so a
// source needs to know nothing about the others before it stores.  The token row is quantised once (int8) or taken as it is (bf16) and stored, with plain
// 16-byte stores, into the receive slab of the rank that owns each of its routes' experts, together with the
// route's scale, local expert id and return address (source rank, flat route).  Same bits as
// quantize_tokens_scatter / gather_rows on one GPU.
template <bool kInt8>
__global__ void __launch_bounds__(256)
peer_dispatch_kernel(const uint16_t* __restrict__ x, const int64_t* __restrict__ topk_ids, int cols, int top_k,
                     const int64_t* __restrict__ dest, const int* __restrict__ route_pos, const int* __restrict__ dest_offsets,
                     int region, PeerSlabLayout slab, const uint64_t* __restrict__ peer_slabs, int rank,
                     int experts_global, int experts_per_rank, int numerics) {
  __shared__ float reduce[32];
  __shared__ int64_t slot_row[32];    // row index in the destination slab, -1 = dropped
  __shared__ uint64_t slot_slab[32];  // base address of the destination slab
  const int64_t token = blockIdx.x;
  if (threadIdx.x < top_k) {
    const int64_t route = token * top_k + threadIdx.x;
    const int64_t d = dest[route];
    const int position = route_pos[route];
    int64_t row = -1;
    uint64_t base = 0;
    if (d >= 0 && position >= 0) {
      row = static_cast<int64_t>(rank) * region + (position - dest_offsets[d]);  // this rank's region of the destination's slab
      base = peer_slabs[d];
    }
    slot_row[threadIdx.x] = row;
    slot_slab[threadIdx.x] = base;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + token * cols);
  const int vec16 = cols >> 4;
  float scale = 1.0f;
  float operand = 1.0f;
  if constexpr (kInt8) {
    float local = 0.0f;
    for (int v = threadIdx.x; v < vec16; v += blockDim.x) {
      float values[16];
      unpack8_bf16(src[2 * v], values);
      unpack8_bf16(src[2 * v + 1], values + 8);
#pragma unroll
      for (int i = 0; i < 16; ++i) local = fmaxf(local, fabsf(values[i]));
    }
    local = warp_max(local);
    if ((threadIdx.x & 31) == 0) reduce[threadIdx.x >> 5] = local;
    __syncthreads();
    float amax = (threadIdx.x & 31) < (blockDim.x >> 5) ? reduce[threadIdx.x & 31] : 0.0f;
    amax = warp_max(amax);
    scale = row_scale_from_amax(amax, numerics);
    operand = quantize_operand(scale, numerics);
  } else {
    __syncthreads();
  }
  if (threadIdx.x < top_k && slot_row[threadIdx.x] >= 0) {
    const int64_t route = token * top_k + threadIdx.x;
    const int64_t row = slot_row[threadIdx.x];
    const uint64_t base = slot_slab[threadIdx.x];
    const int64_t id = topk_ids[route];
    reinterpret_cast<int64_t*>(base + slab.expert)[row] = id >= experts_global ? experts_per_rank : id % experts_per_rank;
    if (kInt8) reinterpret_cast<float*>(base + slab.scale)[row] = scale;
    reinterpret_cast<int2*>(base + slab.source)[row] = make_int2(rank, static_cast<int>(route));
  }
  const int64_t row_bytes = static_cast<int64_t>(cols) * (kInt8 ? 1 : 2);
  for (int v = threadIdx.x; v < vec16; v += blockDim.x) {
    const uint4 a = src[2 * v];
    const uint4 b = src[2 * v + 1];
    uint4 packed = make_uint4(0, 0, 0, 0);
    if constexpr (kInt8) {
      float values[16];
      unpack8_bf16(a, values);
      unpack8_bf16(b, values + 8);
      uint32_t words[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) word |= (static_cast<uint32_t>(quantize_value(values[4 * w + i], operand, numerics)) & 0xffu) << (8 * i);
        words[w] = word;
      }
      packed = make_uint4(words[0], words[1], words[2], words[3]);
    }
    for (int slot = 0; slot < top_k; ++slot) {
      const int64_t row = slot_row[slot];
      if (row < 0) continue;
      uint8_t* out = reinterpret_cast<uint8_t*>(slot_slab[slot] + slab.rows) + row * row_bytes;
      if constexpr (kInt8) {
        reinterpret_cast<uint4*>(out)[v] = packed;
      } else {
        reinterpret_cast<uint4*>(out)[2 * v] = a;
        reinterpret_cast<uint4*>(out)[2 * v + 1] = b;
      }
    }
  }
}

// After the expert rank's route build: the byte address of the fp32 result row of every sorted row, in the
// memory of the rank the route came from.
__global__ void peer_row_ptrs_kernel(const int* __restrict__ sorted_routes, const int* __restrict__ valid_rows, int64_t capacity,
                                     const int2* __restrict__ source, const uint64_t* __restrict__ peer_slabs, size_t route_out_offset,
                                     int row_bytes, uint64_t* __restrict__ row_out_ptrs) {
  const int64_t p = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (p >= capacity || p >= *valid_rows) return;
  const int2 from = source[sorted_routes[p]];
  row_out_ptrs[p] = peer_slabs[from.x] + route_out_offset + static_cast<uint64_t>(from.y) * row_bytes;
}

}  // namespace

cudaError_t launch_peer_barrier(const uint64_t* peer_slabs, const PeerSlabLayout& slab, const int* dest_counts, int world, int rank,
                                unsigned* epoch_counter, int* status, unsigned long long limit_ns, cudaStream_t stream) {
  peer_barrier_kernel<<<1, 64, 0, stream>>>(peer_slabs, slab, dest_counts, world, rank, epoch_counter, status, limit_ns);
  return cudaGetLastError();
}

cudaError_t launch_peer_dispatch(bool int8, const uint16_t* x, const int64_t* topk_ids, int64_t tokens, int cols, int top_k,
                                 const int64_t* dest, const int* route_pos, const int* dest_offsets, int region,
                                 const PeerSlabLayout& slab, const uint64_t* peer_slabs, int rank, int experts_global,
                                 int experts_per_rank, int numerics, cudaStream_t stream) {
  if (tokens <= 0) return cudaSuccess;
  if (int8) {
    peer_dispatch_kernel<true><<<static_cast<unsigned>(tokens), 256, 0, stream>>>(x, topk_ids, cols, top_k, dest, route_pos, dest_offsets,
                                                                                  region, slab, peer_slabs, rank, experts_global,
                                                                                  experts_per_rank, numerics);
  } else {
    peer_dispatch_kernel<false><<<static_cast<unsigned>(tokens), 256, 0, stream>>>(x, topk_ids, cols, top_k, dest, route_pos, dest_offsets,
                                                                                   region, slab, peer_slabs, rank, experts_global,
                                                                                   experts_per_rank, numerics);
  }
  return cudaGetLastError();
}

cudaError_t launch_peer_row_ptrs(const int* sorted_routes, const int* valid_rows, int64_t capacity, const void* source,
                                 const uint64_t* peer_slabs, size_t route_out_offset, int row_bytes, uint64_t* row_out_ptrs,
                                 cudaStream_t stream) {
  if (capacity <= 0) return cudaSuccess;
  peer_row_ptrs_kernel<<<static_cast<unsigned>((capacity + 255) / 256), 256, 0, stream>>>(
      sorted_routes, valid_rows, capacity, static_cast<const int2*>(source), peer_slabs, route_out_offset, row_bytes, row_out_ptrs);
  return cudaGetLastError();
}

cudaError_t launch_dest_ranks(const int64_t* ids, int64_t n, int experts_global, int experts_per_rank, int shared_rank,
                              int64_t* dest, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  dest_ranks_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(ids, n, experts_global, experts_per_rank, shared_rank, dest);
  return cudaGetLastError();
}

cudaError_t launch_local_experts(const int64_t* ids, const int* order, int64_t n, const int* valid_rows, int experts_global,
                                 int experts_per_rank, int64_t* local, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  local_experts_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(ids, order, n, valid_rows, experts_global,
                                                                                experts_per_rank, local);
  return cudaGetLastError();
}

cudaError_t launch_scatter_rows_f32(const float* rows, const int* order, int64_t n, const int* valid_rows, int hidden,
                                    float* route_out, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  scatter_rows_f32_kernel<<<static_cast<unsigned>(n), 256, 0, stream>>>(rows, order, valid_rows, hidden, route_out);
  return cudaGetLastError();
}

}  // namespace fmoe
