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
// first stores a vector of ints into row `rank` of a table in every slab (the per-expert route counts), then
// stores the epoch into its flag in every rank's slab and waits until all flags in its own slab have reached
// that epoch.  The stores of the kernels that ran before it on this stream are complete when it starts (stream
// order), and the fence orders its own stores, so a rank that sees the flag also sees the rows and the table
// row.  The wait is bounded: after limit_ns it records FMOE_ERR_DEVICE_WAIT (detail = the rank it waited for)
// and returns.  What the barrier was meant to guarantee then does not hold, so the caller names the row counts that
// the following stages trust (zero_on_fail, zero_ints of them): they are cleared on expiry and those stages find
// no rows to work on instead of rows that never arrived.
__global__ void __launch_bounds__(256)
peer_barrier_kernel(const uint64_t* __restrict__ peer_slabs, PeerSlabLayout slab, const int* __restrict__ payload, int payload_ints,
                    int world, int rank, unsigned* __restrict__ epoch_counter, int* status, unsigned long long limit_ns,
                    int* __restrict__ zero_on_fail, int zero_ints) {
  __shared__ unsigned epoch_shared;
  __shared__ int expired;
  if (threadIdx.x == 0) expired = 0;
  if (threadIdx.x == 0) {
    epoch_shared = *epoch_counter + 1u;
    *epoch_counter = epoch_shared;
  }
  if (payload != nullptr) {
    const size_t row = slab.counts + sizeof(int) * static_cast<size_t>(rank) * payload_ints;
    for (int i = threadIdx.x; i < world * payload_ints; i += blockDim.x) {
      const int peer = i / payload_ints;
      const int k = i - peer * payload_ints;
      reinterpret_cast<volatile int*>(peer_slabs[peer] + row)[k] = payload[k];
    }
  }
  __threadfence_system();
  __syncthreads();
  const unsigned epoch = epoch_shared;
  const int peer = threadIdx.x;
  if (peer < world) {
    const uint64_t theirs = peer_slabs[peer];
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
        expired = 1;
        break;
      }
    }
  }
  __syncthreads();
  // An error raised earlier on this status block (an earlier barrier of the same call) counts as well.
  if (zero_on_fail != nullptr && (expired || *reinterpret_cast<volatile int*>(status + kStatusError) == FMOE_ERR_DEVICE_WAIT)) {
    for (int i = threadIdx.x; i < zero_ints; i += blockDim.x) zero_on_fail[i] = 0;
  }
}

// After the count exchange every rank holds C[source][expert] for all experts (experts_total = routed experts
// + 1 if there is a shared expert, whose routes stay on their own rank).  The rows of one expert lie together at
// its owner, sources in rank order, experts in local order (the shared expert last); from C every rank computes
//   send_base[e]    where this rank's rows for expert e start in the owner's slab, and, as an owner,
//   local_counts / local_offsets of its own experts (offsets[local_experts] = rows received in all).
// One block.
__global__ void __launch_bounds__(1024)
peer_layout_kernel(const int* __restrict__ count_matrix, int row_stride, int world, int rank, int experts_global, int per_rank,
                   int has_shared, int* __restrict__ send_base, int* __restrict__ local_counts, int* __restrict__ local_offsets,
                   const int* __restrict__ status) {
  extern __shared__ int layout_smem[];
  const int experts_total = experts_global + (has_shared ? 1 : 0);
  if (status[kStatusError] == FMOE_ERR_DEVICE_WAIT) {
    // The count exchange gave up: a row of the table may be missing or half written.  Nothing is sent and nothing
    // is expected (the dispatch kernel checks the same word).
    const int local_experts = per_rank + (has_shared ? 1 : 0);
    for (int e = threadIdx.x; e < experts_total; e += blockDim.x) send_base[e] = 0;
    for (int le = threadIdx.x; le <= local_experts; le += blockDim.x) {
      if (le < local_experts) local_counts[le] = 0;
      local_offsets[le] = 0;
    }
    return;
  }
  int* total = layout_smem;                  // rows of expert e at its owner
  int* before_me = total + experts_total;    // rows of expert e from lower source ranks
  int* scan = before_me + experts_total;     // exclusive scan of total[] over the routed experts (+ end)
  for (int e = threadIdx.x; e < experts_total; e += blockDim.x) {
    int sum = 0, lower = 0;
    if (e < experts_global) {
      for (int s = 0; s < world; ++s) {
        const int c = count_matrix[s * row_stride + e];
        if (s < rank) lower += c;
        sum += c;
      }
    } else {
      sum = count_matrix[rank * row_stride + e];  // the shared expert: only this rank's own routes, kept here
    }
    total[e] = sum;
    before_me[e] = lower;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // exclusive scan over the routed experts, 32 per step
    int carry = 0;
    for (int base = 0; base < experts_global; base += 32) {
      const int e = base + threadIdx.x;
      const int value = e < experts_global ? total[e] : 0;
      int inclusive = value;
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const int other = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if (threadIdx.x >= offset) inclusive += other;
      }
      if (e < experts_global) scan[e] = carry + inclusive - value;
      carry += __shfl_sync(0xffffffffu, inclusive, 31);
    }
    if (threadIdx.x == 0) scan[experts_global] = carry;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts_total; e += blockDim.x) {
    if (e < experts_global) {
      const int owner = e / per_rank;
      send_base[e] = scan[e] - scan[owner * per_rank] + before_me[e];
    } else {
      send_base[e] = scan[(rank + 1) * per_rank] - scan[rank * per_rank];  // after this rank's routed experts
    }
  }
  const int local_experts = per_rank + (has_shared ? 1 : 0);
  for (int le = threadIdx.x; le <= local_experts; le += blockDim.x) {
    const int first = rank * per_rank;
    const int routed_end = scan[first + per_rank] - scan[first];
    if (le < per_rank) {
      local_counts[le] = total[first + le];
      local_offsets[le] = scan[first + le] - scan[first];
    } else if (le == per_rank && has_shared) {
      local_counts[le] = total[experts_global];
      local_offsets[le] = routed_end;
    }
    if (le == local_experts) local_offsets[le] = routed_end + (has_shared ? total[experts_global] : 0);
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

// One CTA per token.  send_base[e] is where this rank's rows for expert e start in the owner's slab (see
// peer_layout_kernel), so every row lands at its final, expert-sorted position.  The token row is quantised once (int8) or taken as it is (bf16) and stored, with plain
// 16-byte stores, into the receive slab of the rank that owns each of its routes' experts, together with the
// route's scale, local expert id and return address (source rank, flat route).  Same bits as
// quantize_tokens_scatter / gather_rows on one GPU.
template <bool kInt8>
__global__ void __launch_bounds__(256)
peer_dispatch_kernel(const uint16_t* __restrict__ x, const int64_t* __restrict__ topk_ids, int cols, int top_k,
                     const int* __restrict__ route_pos, const int* __restrict__ expert_offsets, const int* __restrict__ send_base,
                     PeerSlabLayout slab, const uint64_t* __restrict__ peer_slabs, int rank, int experts_global, int experts_per_rank,
                     int has_shared, int numerics, int64_t capacity, int* __restrict__ status) {
  __shared__ float reduce[32];
  __shared__ int64_t slot_row[32];    // row index in the destination slab, -1 = dropped
  __shared__ uint64_t slot_slab[32];  // base address of the destination slab
  const int64_t token = blockIdx.x;
  if (status[kStatusError] == FMOE_ERR_DEVICE_WAIT) return;  // the count exchange gave up: no destination is known
  if (threadIdx.x < top_k) {
    const int64_t route = token * top_k + threadIdx.x;
    const int64_t id = topk_ids[route];
    const int position = route_pos[route];  // position in this rank's expert-sorted route list, -1 = dropped
    int64_t row = -1;
    uint64_t base = 0;
    if (position >= 0) {
      const int e = static_cast<int>(id);
      const int owner = (has_shared && e == experts_global) ? rank : e / experts_per_rank;
      row = send_base[e] + (position - expert_offsets[e]);
      base = peer_slabs[owner];
      if (row < 0 || row >= capacity) {
        // Cannot happen with a consistent count table (capacity is every route of every rank); a torn table must
        // not turn into a store outside the slab.
        raise_error(status, FMOE_ERR_DEVICE_WAIT, -1);
        row = -1;
      }
    }
    slot_row[threadIdx.x] = row;
    slot_slab[threadIdx.x] = base;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + token * cols);
  const int vec16 = cols >> 4;
  float scale = 1.0f;
  float operand = 1.0f;
  float inverse = 1.0f;
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
    inverse = __fdiv_rn(1.0f, scale);
  } else {
    __syncthreads();
  }
  if (threadIdx.x < top_k && slot_row[threadIdx.x] >= 0) {
    const int64_t route = token * top_k + threadIdx.x;
    const int64_t row = slot_row[threadIdx.x];
    const uint64_t base = slot_slab[threadIdx.x];
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
        if (numerics == FMOE_NUMERICS_TORCHREF) {
          words[w] = quantize4_torchref_fast(values + 4 * w, operand, inverse);
          continue;
        }
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          word |= (static_cast<uint32_t>(quantize_value(values[4 * w + i], operand, numerics)) & 0xffu) << (8 * i);
        }
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

// The byte address of the result row of every received row, in the memory of the rank the route came from.
// A return address that does not name a rank of the box and one of its routes (a row that never arrived: the slab
// starts zeroed, and a failed barrier leaves old rows behind) is reported and replaced by the local scrap row, so
// that the down GEMM's epilogue never stores through it.
__global__ void peer_row_ptrs_kernel(const int* __restrict__ valid_rows, int64_t capacity,
                                     const int2* __restrict__ source, const uint64_t* __restrict__ peer_slabs, size_t route_out_offset,
                                     int row_bytes, uint64_t* __restrict__ row_out_ptrs, int world, int64_t routes_max, uint64_t scrap_row,
                                     int* __restrict__ status) {
  const int64_t p = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (p >= capacity || p >= *valid_rows) return;
  const int2 from = source[p];
  if (from.x < 0 || from.x >= world || from.y < 0 || from.y >= routes_max) {
    raise_error(status, FMOE_ERR_DEVICE_WAIT, -2);
    row_out_ptrs[p] = scrap_row;
    return;
  }
  row_out_ptrs[p] = peer_slabs[from.x] + route_out_offset + static_cast<uint64_t>(from.y) * row_bytes;
}

}  // namespace

cudaError_t launch_peer_barrier(const uint64_t* peer_slabs, const PeerSlabLayout& slab, const int* payload, int payload_ints, int world,
                                int rank, unsigned* epoch_counter, int* status, unsigned long long limit_ns, cudaStream_t stream,
                                int* zero_on_fail, int zero_ints) {
  peer_barrier_kernel<<<1, 256, 0, stream>>>(peer_slabs, slab, payload, payload_ints, world, rank, epoch_counter, status, limit_ns,
                                             zero_on_fail, zero_ints);
  return cudaGetLastError();
}

cudaError_t launch_peer_layout(const int* count_matrix, int world, int rank, int experts_global, int per_rank, int has_shared,
                               int row_stride, int* send_base, int* local_counts, int* local_offsets, const int* status,
                               cudaStream_t stream) {
  const size_t smem = (3 * static_cast<size_t>(experts_global + 1) + 1) * sizeof(int);
  peer_layout_kernel<<<1, 1024, smem, stream>>>(count_matrix, row_stride, world, rank, experts_global, per_rank, has_shared, send_base,
                                                local_counts, local_offsets, status);
  return cudaGetLastError();
}

cudaError_t launch_peer_dispatch(bool int8, const uint16_t* x, const int64_t* topk_ids, int64_t tokens, int cols, int top_k,
                                 const int* route_pos, const int* expert_offsets, const int* send_base, const PeerSlabLayout& slab,
                                 const uint64_t* peer_slabs, int rank, int experts_global, int experts_per_rank, int has_shared,
                                 int numerics, int64_t capacity, int* status, cudaStream_t stream) {
  if (tokens <= 0) return cudaSuccess;
  if (int8) {
    peer_dispatch_kernel<true><<<static_cast<unsigned>(tokens), 256, 0, stream>>>(x, topk_ids, cols, top_k, route_pos, expert_offsets, send_base,
                                                                                  slab, peer_slabs, rank, experts_global, experts_per_rank,
                                                                                  has_shared, numerics, capacity, status);
  } else {
    peer_dispatch_kernel<false><<<static_cast<unsigned>(tokens), 256, 0, stream>>>(x, topk_ids, cols, top_k, route_pos, expert_offsets, send_base,
                                                                                   slab, peer_slabs, rank, experts_global, experts_per_rank,
                                                                                   has_shared, numerics, capacity, status);
  }
  return cudaGetLastError();
}

cudaError_t launch_peer_row_ptrs(const int* valid_rows, int64_t capacity, const void* source, const uint64_t* peer_slabs,
                                 size_t route_out_offset, int row_bytes, uint64_t* row_out_ptrs, int world, int64_t routes_max,
                                 void* scrap_row, int* status, cudaStream_t stream) {
  if (capacity <= 0) return cudaSuccess;
  peer_row_ptrs_kernel<<<static_cast<unsigned>((capacity + 255) / 256), 256, 0, stream>>>(
      valid_rows, capacity, static_cast<const int2*>(source), peer_slabs, route_out_offset, row_bytes, row_out_ptrs, world, routes_max,
      reinterpret_cast<uint64_t>(scrap_row), status);
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
