// Route build: per-expert route lists and the work-item lists of the grouped GEMMs.
//
// The reference walks topk_ids once on the calling thread and pushes each flat route id t*K+slot
// onto its expert's vector (csrc/moe/arm/i8mm_w8a8/kernels.cpp:583-592;
// csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:6455-6469), i.e. a stable counting sort by expert.
// Here the same order is produced by three small kernels built on warp primitives:
//   1. route_hist:    every warp owns a unit of kUnitRoutes consecutive routes and histograms it;
//   2. route_scan:    one block turns the unit histograms into per-(unit, expert) cursors, the
//                     per-expert offsets and the (expert, row-tile) work items;
//   3. route_scatter: every warp replays its unit in order; __match_any_sync ranks equal ids inside
//                     a 32-route round, so positions are assigned in ascending flat-id order.
// Ids outside [0, E) raise FMOE_ERR_EXPERT_ID_RANGE in the status block and are dropped.
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace fmoe {

namespace {

constexpr int kWarpsPerBlock = 4;

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
route_hist_kernel(const int64_t* __restrict__ topk_ids, int64_t routes, int experts, int units, int* unit_hist, int* status) {
  extern __shared__ int smem_hist[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * kWarpsPerBlock + warp;
  int* hist = smem_hist + warp * experts;
  for (int e = lane; e < experts; e += 32) hist[e] = 0;
  __syncwarp();
  if (unit >= units) return;
  const int64_t begin = static_cast<int64_t>(unit) * kUnitRoutes;
  for (int round = 0; round < kUnitRoutes / 32; ++round) {
    const int64_t route = begin + round * 32 + lane;
    if (route < routes) {
      const int64_t id = topk_ids[route];
      if (id < 0 || id >= experts) {
        raise_error(status, FMOE_ERR_EXPERT_ID_RANGE, static_cast<int>(route));
      } else {
        atomicAdd(hist + id, 1);
      }
    }
  }
  __syncwarp();
  for (int e = lane; e < experts; e += 32) unit_hist[static_cast<int64_t>(unit) * experts + e] = hist[e];
}

// Exclusive scan of `values[0..n)` by one warp, 32 entries per step; returns the total.
__device__ int warp_exclusive_scan(const int* values, int* out, int n, int lane) {
  int carry = 0;
  for (int base = 0; base < n; base += 32) {
    const int index = base + lane;
    const int value = index < n ? values[index] : 0;
    int inclusive = value;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, inclusive, offset);
      if (lane >= offset) inclusive += other;
    }
    if (index < n) out[index] = carry + inclusive - value;
    carry += __shfl_sync(0xffffffffu, inclusive, 31);
  }
  return carry;
}

// Work items: (expert, first sorted row, rows, group key) for every row tile of every active expert, and the
// number of active experts.  Lists a and b (gate_up and down GEMM) have independent tile heights.  With
// split_rows > 0 they hold only the experts with at most split_rows rows, and lists c and d (tile big_tile) the
// experts with more: the batch's routing decides on the device, expert by expert, whether an expert's rows go to
// the weight-streaming kernel or to the two-SM kernel, with no host-side guess about the distribution.
// Called by a whole block; scan_tmp has room for 2 * experts + 1 ints (global or shared).
__device__ void build_items(int experts, const int* counts, const int* offsets, const ItemLists& lists, int* scan_tmp, int* status) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int split_rows = lists.split_rows;
  const int max_items = lists.max_items;
  for (int list = 0; list < 4; ++list) {
    const bool big = list >= 2;
    const int word = list == 0 ? kStatusItems : list == 1 ? kStatusItemsB : list == 2 ? kStatusItemsC : kStatusItemsD;
    if (big && split_rows <= 0) {
      if (threadIdx.x == 0) status[word] = 0;
      continue;
    }
    const int tile = list == 0 ? lists.tile_a : list == 1 ? lists.tile_b : lists.big_tile;
    int* items = list == 0 ? lists.items_a : list == 1 ? lists.items_b : list == 2 ? lists.items_c : lists.items_d;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
      const bool mine = split_rows <= 0 || (big ? counts[e] > split_rows : counts[e] <= split_rows);
      scan_tmp[e] = mine ? (counts[e] + tile - 1) / tile : 0;
    }
    __syncthreads();
    if (warp == 0) {
      const int total = warp_exclusive_scan(scan_tmp, scan_tmp + experts, experts, lane);
      if (lane == 0) status[word] = total < max_items ? total : max_items;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
      const int tiles = scan_tmp[e];
      const int first = scan_tmp[experts + e];
      // The expert's rows are spread evenly over its tiles (in steps of 32 rows, the granularity of the MMA's N):
      // 290 rows become 160 + 130, not 256 + 34.
      int rows_per = tile;
      if (tiles > 1) {
        const int step = tile < 32 ? tile : 32;
        const int even = ((counts[e] + tiles - 1) / tiles + step - 1) / step * step;
        if (even <= tile && (tiles - 1) * even < counts[e]) rows_per = even;
      }
      for (int t = 0; t < tiles && first + t < max_items; ++t) {
        int* item = items + 4 * static_cast<int64_t>(first + t);
        item[0] = e;
        item[1] = offsets[e] + t * rows_per;
        item[2] = min(rows_per, counts[e] - t * rows_per);
        // Group key for the unit order of the grouped GEMM: first item of this expert and its tile count, so
        // that the row tiles of one (expert, channel block) are consecutive work units (see decode_unit).
        item[3] = tiles < 2048 ? (first | (tiles << 20)) : ((first + t) | (1 << 20));
      }
    }
    __syncthreads();
  }
  if (warp == 0) {
    int active = 0;
    for (int e = lane; e < experts; e += 32) active += counts[e] > 0;
    active = warp_sum(active);
    if (lane == 0) status[kStatusActive] = active;
  }
}

// The whole route build in one block for lists of at most kSmallRoutes entries (decode batches, and the
// expert-parallel lists at decode): ids and histogram in shared memory, the stable position of a route is its
// expert's offset plus the number of earlier routes with the same id (a scan of the shared ids, at most
// kSmallRoutes steps).  Same outputs as the three-kernel form.
constexpr int kSmallRoutes = 1024;

__global__ void __launch_bounds__(kSmallRoutes)
route_small_kernel(const int64_t* __restrict__ topk_ids, int routes, int experts, ItemLists lists, int* status, int* counts, int* offsets,
                   int* sorted_routes, int* row_expert, int* route_pos) {
  extern __shared__ int small_smem[];
  int* s_id = small_smem;
  int* s_counts = s_id + kSmallRoutes;
  int* s_offsets = s_counts + experts;
  int* s_tmp = s_offsets + experts + 1;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) s_counts[e] = 0;
  __syncthreads();
  const int r = threadIdx.x;
  int id = -1;
  if (r < routes) {
    const int64_t value = topk_ids[r];
    if (value >= 0 && value < experts) {
      id = static_cast<int>(value);
      atomicAdd(s_counts + id, 1);
    } else {
      raise_error(status, FMOE_ERR_EXPERT_ID_RANGE, r);
    }
  }
  s_id[r] = id;
  __syncthreads();
  if (warp == 0) {
    const int total = warp_exclusive_scan(s_counts, s_offsets, experts, lane);
    if (lane == 0) s_offsets[experts] = total;
  }
  __syncthreads();
  int position = -1;
  if (id >= 0) {
    int rank = 0;
    for (int j = 0; j < r; ++j) rank += s_id[j] == id;
    position = s_offsets[id] + rank;
    sorted_routes[position] = r;
    row_expert[position] = id;
  }
  if (route_pos != nullptr && r < routes) route_pos[r] = position;
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) {
    if (e < experts) counts[e] = s_counts[e];
    offsets[e] = s_offsets[e];
  }
  build_items(experts, s_counts, s_offsets, lists, s_tmp, status);
}

__global__ void __launch_bounds__(1024)
route_scan_kernel(int experts, int units, int* unit_hist, int* counts, int* offsets, ItemLists lists, int* scan_tmp, int* status) {
  // Pass 1: per expert, exclusive scan over units (unit_hist becomes the unit's cursor relative to the
  // expert's first row) and the expert total.  One thread per expert (adjacent threads read adjacent words);
  // the units are taken sixteen at a time, all loads of a batch issued before the first store, so the
  // sweep costs one memory round trip per batch and not one per unit.
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kBatch = 16;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int running = 0;
    for (int base = 0; base < units; base += kBatch) {
      int values[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        const int u = base + i;
        values[i] = u < units ? unit_hist[static_cast<int64_t>(u) * experts + e] : 0;
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        const int u = base + i;
        if (u < units) unit_hist[static_cast<int64_t>(u) * experts + e] = running;
        running += values[i];
      }
    }
    counts[e] = running;
  }
  __syncthreads();
  if (warp == 0) {
    const int total = warp_exclusive_scan(counts, offsets, experts, lane);
    if (lane == 0) offsets[experts] = total;
  }
  __syncthreads();
  build_items(experts, counts, offsets, lists, scan_tmp, status);
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
route_scatter_kernel(const int64_t* __restrict__ topk_ids, int64_t routes, int experts, int units,
                     const int* __restrict__ unit_hist, const int* __restrict__ offsets, int* sorted_routes,
                     int* row_expert, int* route_pos) {
  extern __shared__ int smem_cursor[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * kWarpsPerBlock + warp;
  if (unit >= units) return;
  int* cursor = smem_cursor + warp * experts;
  for (int e = lane; e < experts; e += 32) cursor[e] = offsets[e] + unit_hist[static_cast<int64_t>(unit) * experts + e];
  __syncwarp();
  const int64_t begin = static_cast<int64_t>(unit) * kUnitRoutes;
  const unsigned lanes_below = (1u << lane) - 1u;
  for (int round = 0; round < kUnitRoutes / 32; ++round) {
    const int64_t route = begin + round * 32 + lane;
    int id = -1;
    if (route < routes) {
      const int64_t value = topk_ids[route];
      if (value >= 0 && value < experts) id = static_cast<int>(value);
    }
    const unsigned peers = __match_any_sync(0xffffffffu, id);
    int position = -1;
    if (id >= 0) position = cursor[id] + __popc(peers & lanes_below);
    __syncwarp();
    if (id >= 0 && (peers & lanes_below) == 0) cursor[id] += __popc(peers);
    __syncwarp();
    if (id >= 0) {
      sorted_routes[position] = static_cast<int>(route);
      row_expert[position] = id;
    }
    // Inverse permutation: sorted position of every flat route (-1 for a dropped route).
    if (route_pos != nullptr && route < routes) route_pos[route] = position;
  }
}

}  // namespace

size_t route_scratch_bytes(int64_t routes, int experts) {
  const int64_t units = (routes + kUnitRoutes - 1) / kUnitRoutes;
  return static_cast<size_t>((units > 0 ? units : 1) * experts + 2 * (experts + 1)) * sizeof(int);
}

cudaError_t launch_route_build(const int64_t* topk_ids, int64_t routes, int experts, const ItemLists& lists, int* status, int* counts,
                               int* offsets, int* sorted_routes, int* row_expert, int* scratch, cudaStream_t stream, int* route_pos) {
  if (routes <= kSmallRoutes) {
    const size_t small_bytes = (static_cast<size_t>(kSmallRoutes) + 4 * static_cast<size_t>(experts) + 4) * sizeof(int);
    route_small_kernel<<<1, kSmallRoutes, small_bytes, stream>>>(topk_ids, static_cast<int>(routes), experts, lists, status, counts, offsets,
                                                                 sorted_routes, row_expert, route_pos);
    return cudaGetLastError();
  }
  const int units = static_cast<int>((routes + kUnitRoutes - 1) / kUnitRoutes);
  int* unit_hist = scratch;
  int* scan_tmp = scratch + static_cast<int64_t>(units > 0 ? units : 1) * experts;
  const size_t smem = static_cast<size_t>(kWarpsPerBlock) * experts * sizeof(int);
  const int blocks = (units + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0) {
    route_hist_kernel<<<blocks, kWarpsPerBlock * 32, smem, stream>>>(topk_ids, routes, experts, units, unit_hist, status);
  }
  route_scan_kernel<<<1, 1024, 0, stream>>>(experts, units, unit_hist, counts, offsets, lists, scan_tmp, status);
  if (blocks > 0) {
    route_scatter_kernel<<<blocks, kWarpsPerBlock * 32, smem, stream>>>(topk_ids, routes, experts, units, unit_hist,
                                                                        offsets, sorted_routes, row_expert, route_pos);
  }
  return cudaGetLastError();
}

namespace {
// Work items and the status words of the grouped GEMMs from given per-expert counts and offsets (rows that
// already lie in expert order: nothing to sort).
__global__ void __launch_bounds__(1024)
items_from_counts_kernel(int experts, const int* __restrict__ counts, const int* __restrict__ offsets, ItemLists lists, int* scan_tmp,
                         int* status) {
  build_items(experts, counts, offsets, lists, scan_tmp, status);
}

}  // namespace

cudaError_t launch_items_from_counts(int experts, const int* counts, const int* offsets, const ItemLists& lists, int* scratch, int* status,
                                     cudaStream_t stream) {
  items_from_counts_kernel<<<1, 1024, 0, stream>>>(experts, counts, offsets, lists, scratch, status);
  return cudaGetLastError();
}


// ---- allocation-free route build ---------------------------------------------------------------
//
// Some hosts of this library must not allocate device memory once they are serving: an inference
// server that handed the whole HBM budget to its KV-cache pool at start-up has nothing left for a
// cudaMalloc to take, and a runtime whose memory plan is frozen after warm-up treats any later
// allocation as a bug.  For them the route build is also offered with its scratch (the per-unit
// histograms, the scan temporaries and the status block) in a fixed array that lives in the
// library's device image, so the call needs no workspace and performs no allocation of any kind.
// The price is a fixed ceiling on the problem size and one array shared by every call.

namespace {

constexpr int64_t kStaticMaxRoutes = 131072;  // tokens * top_k
constexpr int kStaticMaxExperts = 512;
constexpr size_t kStaticScratchInts = fmoe::kStatusWords + static_cast<size_t>(kStaticMaxRoutes / fmoe::kUnitRoutes) * kStaticMaxExperts +
                                      2 * (kStaticMaxExperts + 1);
constexpr int kStaticMaxDevices = 64;

// 528 KB per GPU, held from the moment the library is loaded on that GPU until the process exits.
static __device__ __align__(256) int g_static_route_scratch[kStaticScratchInts];

// In host code the array's name only stands for the symbol; the address a kernel can use has to be
// asked for, per device, with that device current.
int* static_scratch_for_current_device(cudaError_t* error) {
  static std::mutex guard;
  static int* address[kStaticMaxDevices] = {};
  int device = 0;
  *error = cudaGetDevice(&device);
  if (*error != cudaSuccess) return nullptr;
  if (device < 0 || device >= kStaticMaxDevices) {
    *error = cudaErrorInvalidDevice;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(guard);
  if (address[device] == nullptr) {
    int* pointer = nullptr;
    *error = cudaGetSymbolAddress(reinterpret_cast<void**>(&pointer), g_static_route_scratch);
    if (*error != cudaSuccess) return nullptr;
    address[device] = pointer;
  }
  return address[device];
}

}  // namespace

}  // namespace fmoe

extern "C" int fmoe_route_build_noalloc(const int64_t* topk_ids, int64_t tokens, int32_t top_k, int32_t experts, int32_t* counts,
                                        int32_t* offsets, int32_t* sorted_routes, int32_t* row_expert, int32_t* status_out,
                                        void* stream_ptr) {
  char text[256];
  if (tokens < 0 || top_k <= 0 || experts <= 0) return fmoe::report_error(FMOE_ERR_INVALID_ARGUMENT, "invalid route-build shape");
  const int64_t routes = tokens * top_k;
  if (routes > fmoe::kStaticMaxRoutes || experts > fmoe::kStaticMaxExperts) {
    snprintf(text, sizeof(text),
             "fmoe_route_build_noalloc: %lld routes x %d experts exceeds the static scratch (at most %lld routes and %d experts); "
             "use fmoe_w8a8_forward / fmoe_bf16_forward with a caller workspace for larger problems",
             static_cast<long long>(routes), experts, static_cast<long long>(fmoe::kStaticMaxRoutes), fmoe::kStaticMaxExperts);
    return fmoe::report_error(FMOE_ERR_INVALID_ARGUMENT, text);
  }
  if (counts == nullptr || offsets == nullptr || status_out == nullptr ||
      (routes > 0 && (topk_ids == nullptr || sorted_routes == nullptr || row_expert == nullptr))) {
    return fmoe::report_error(FMOE_ERR_INVALID_ARGUMENT, "fmoe_route_build_noalloc: null pointer");
  }
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || !fmoe_device_supported(device)) {
    return fmoe::report_error(FMOE_ERR_UNSUPPORTED_DEVICE, "fmoe_route_build_noalloc: the current device is not a compute capability 10.x GPU");
  }
  cudaError_t error = cudaSuccess;
  int* scratch = fmoe::static_scratch_for_current_device(&error);
  if (scratch == nullptr) {
    snprintf(text, sizeof(text), "fmoe_route_build_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(error));
    return fmoe::report_error(FMOE_ERR_CUDA, text);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  int* status = scratch;                       // kStatusWords ints: must start at zero, the kernels only ever raise it
  int* work = scratch + fmoe::kStatusWords;    // histograms + scan temporaries: fully rewritten by every call
  error = cudaMemsetAsync(status, 0, sizeof(int) * fmoe::kStatusWords, stream);
  if (error == cudaSuccess) {
    error = fmoe::launch_route_build(topk_ids, routes, experts, fmoe::no_item_lists(), status, counts, offsets, sorted_routes, row_expert, work,
                                     stream);
  }
  if (error == cudaSuccess) error = cudaMemcpyAsync(status_out, status, 2 * sizeof(int), cudaMemcpyDeviceToDevice, stream);
  if (error != cudaSuccess) {
    snprintf(text, sizeof(text), "fmoe_route_build_noalloc: %s", cudaGetErrorString(error));
    return fmoe::report_error(FMOE_ERR_CUDA, text);
  }
  return FMOE_OK;
}
