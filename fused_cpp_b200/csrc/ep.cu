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

}  // namespace

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
