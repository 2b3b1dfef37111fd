// Grouped expert GEMM, two-SM form: a cluster of two CTAs drives `tcgen05.mma.cta_group::2` so that a
// 256 (channels) x 256 (tokens) tile costs each SM only 128 + 128 operand rows per K step.
//
// Same work as umma_gemm.cu (the reference's two run_stage sweeps and their epilogues,
// csrc/moe/arm/i8mm_w8a8/kernels.cpp:328-368, 230-257) for the prefill regime, where an expert has
// hundreds of rows and the one-SM kernel is limited by operand delivery from L2: a 128x128 tile needs
// 96 bytes of shared-memory fill per tensor-core clock, this one needs 64, and every weight byte is
// read once per 256 rows instead of once per 128.
//
// Pair layout.  CTA r of the pair (r = 0 leads) stages its own halves: 128 A rows (weight channels)
// and 128 B rows (tokens); the MMA reads A rows 0..127 from CTA 0 and 128..255 from CTA 1, B likewise,
// and leaves D rows 128r..128r+127 x 256 token columns in CTA r's tensor memory.
//   down:    A rows of CTA r = channels n0 + 128 r .. + 127.
//   gate_up: A rows of CTA r = gate channels c0 + 64 r .. + 63 followed by the up channels of the same
//            indices (two 64-row TMA loads), so each CTA holds gate and up of its 64 channels; the
//            epilogue's gate warps (TMEM lanes 0..63) and up warps (lanes 64..127) swap half of their
//            columns through shared memory and each finish half of the SwiGLU outputs.
// Barriers.  Both producers signal the leader's "full" barrier (TMA complete_tx through the cluster
// address), the leader's single MMA thread commits to the "empty" and "accumulator full" barriers of
// both CTAs, and the follower's epilogue warps arrive on the leader's "accumulator empty" barrier
// through its cluster address.  No load is a multicast load.  Every wait is bounded (see ptx.cuh).
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace fmoe {

namespace {

constexpr int kRowsPerCta = 128;    // A rows and B rows staged by one CTA
constexpr int kPairTokens = 256;    // MMA N
constexpr int kBlockKBytes = 128;
constexpr int kUmmaKBytes = 32;
constexpr int kThreads = 192;
constexpr int kStages = 6;
constexpr int kStageBytes = 2 * kRowsPerCta * kBlockKBytes;  // 32 KB
constexpr int kAccColumns = kPairTokens;                     // one accumulator: 256 columns
constexpr int kTmemColumns = 512;                            // two accumulators
constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kStageBytes + 8192;

// Per-column values of the current work unit, staged once so that the element loop reads shared memory.
struct ColumnMeta {
  float scale[256];
  int target[256];
};

struct PairControl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  uint32_t exchange[2][64][4];  // [gate->up | up->gate][channel][column]
  ColumnMeta meta[2];
};

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_address, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_address), "r"(cta));
  return remote;
}

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}

// TMA tiled load whose completion bytes go to an mbarrier given by its cluster address (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_address, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(ptx::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_address), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(smem_result)), "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

// One arrival on the mbarrier at `cluster_address` once every MMA issued so far by this thread is done.
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t cluster_address) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_address) : "memory");
}

template <bool kInt8>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  if constexpr (kInt8) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <bool kInt8, bool kGateUp, bool kDense>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
umma_pair_grouped_gemm_kernel(const __grid_constant__ CUtensorMap weight_map, const __grid_constant__ CUtensorMap token_map,
                              GroupedGemmArgs args) {
  constexpr int kElemBytes = kInt8 ? 1 : 2;
  constexpr int kBlockKElems = kBlockKBytes / kElemBytes;
  constexpr int kChannelsPerUnit = kGateUp ? 128 : 256;  // output channels one pair finishes per work unit

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  PairControl* ctl = reinterpret_cast<PairControl*>(smem + static_cast<size_t>(kStages) * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_cta_rank();
  const bool leader = cta == 0;
  int* status = args.status_rw;

  const int items = min(args.status[args.item_count_word], args.max_items);
  const int n_blocks = (args.n_out + kChannelsPerUnit - 1) / kChannelsPerUnit;
  const int n_total = kGateUp ? 2 * args.n_out : args.n_out;
  const int64_t units = static_cast<int64_t>(items) * n_blocks;
  const int k_blocks = (args.k + kBlockKElems - 1) / kBlockKElems;
  const int64_t first_unit = blockIdx.x >> 1;
  const int64_t unit_stride = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&ctl->acc_full[b], 1);
      ptx::mbar_init(&ctl->acc_empty[b], 8);  // four epilogue warps in each CTA of the pair
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, kTmemColumns);
    tmem_relinquish_pair();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  cluster_sync();  // the peer's barriers are initialised before anything signals them
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      ptx::prefetch_tensormap(&weight_map);
      ptx::prefetch_tensormap(&token_map);
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      for (int64_t unit = first_unit; unit < units; unit += unit_stride) {
        int item, block;
        decode_unit(args.items, unit, n_blocks, &item, &block);
        const int c0 = block * kChannelsPerUnit;
        const int expert = args.items[4 * item + 0];
        const int row0 = args.items[4 * item + 1];
        const int weight_row = expert * n_total + c0;
        // The MMA takes the first N/2 token rows from the leader's tile and the other N/2 from the follower's.
        const int mma_n = min(kPairTokens, (args.items[4 * item + 2] + 31) & ~31);
        const int token_row = row0 + (mma_n / 2) * static_cast<int>(cta);
        for (int kb = 0; kb < k_blocks; ++kb) {
          ptx::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag, status, 11);
          uint8_t* stage_base = smem + static_cast<size_t>(stage) * kStageBytes;
          const uint32_t full_leader = map_to_cta(ptx::smem_u32(&ctl->full[stage]), 0);
          if (leader) ptx::mbar_arrive_expect_tx(&ctl->full[stage], 2 * kStageBytes);
          const int x = kb * kBlockKElems;
          if (kGateUp) {
            tma_load_2d_pair(stage_base, &weight_map, full_leader, x, weight_row + 64 * static_cast<int>(cta));
            tma_load_2d_pair(stage_base + 64 * kBlockKBytes, &weight_map, full_leader, x, weight_row + args.n_out + 64 * static_cast<int>(cta));
          } else {
            tma_load_2d_pair(stage_base, &weight_map, full_leader, x, weight_row + kRowsPerCta * static_cast<int>(cta));
          }
          tma_load_2d_pair(stage_base + kRowsPerCta * kBlockKBytes, &token_map, full_leader, x, token_row);
          ++issued;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (leader) {
        // Drain: the leader's full barriers count both CTAs' bytes, so this also covers the follower's loads.
        const int pending = issued < kStages ? issued : kStages;
        for (int back = 0; back < pending; ++back) {
          int s = stage - 1 - back;
          uint32_t p = phase;
          if (s < 0) {
            s += kStages;
            p ^= 1u;
          }
          const unsigned long long start = ptx::global_timer_ns();
          while (!ptx::mbar_try_wait(&ctl->full[s], p)) {
            if (ptx::global_timer_ns() - start > ptx::kWaitLimitNs) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      for (int64_t unit = first_unit; unit < units; unit += unit_stride, ++local) {
        const int buffer = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        // N follows the rows this unit really has (a multiple of 32 for two-SM MMAs).
        int item, block;
        decode_unit(args.items, unit, n_blocks, &item, &block);
        const int item_rows = args.items[4 * item + 2];
        const int mma_n = min(kPairTokens, (item_rows + 31) & ~31);
        const uint32_t idesc = ptx::make_instr_desc(kInt8, 2 * kRowsPerCta, mma_n);
        ptx::mbar_wait(&ctl->acc_empty[buffer], (use & 1u) ^ 1u, abort_flag, status, 12);
        ptx::tcgen05_fence_after();
        const uint32_t acc = tmem_base + static_cast<uint32_t>(buffer * kAccColumns);
        for (int kb = 0; kb < k_blocks; ++kb) {
          ptx::mbar_wait(&ctl->full[stage], phase, abort_flag, status, 13);
          ptx::tcgen05_fence_after();
          const uint32_t stage_addr = ptx::smem_u32(smem + static_cast<size_t>(stage) * kStageBytes);
#pragma unroll
          for (int ks = 0; ks < kBlockKBytes / kUmmaKBytes; ++ks) {
            const uint64_t desc_a = ptx::make_smem_desc_sw128(stage_addr + ks * kUmmaKBytes);
            const uint64_t desc_b = ptx::make_smem_desc_sw128(stage_addr + kRowsPerCta * kBlockKBytes + ks * kUmmaKBytes);
            umma_pair<kInt8>(acc, desc_a, desc_b, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
          }
          const uint32_t empty_local = ptx::smem_u32(&ctl->empty[stage]);
          tcgen05_commit_pair(map_to_cta(empty_local, 0));
          tcgen05_commit_pair(map_to_cta(empty_local, 1));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        const uint32_t full_local = ptx::smem_u32(&ctl->acc_full[buffer]);
        tcgen05_commit_pair(map_to_cta(full_local, 0));
        tcgen05_commit_pair(map_to_cta(full_local, 1));
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
    const int quarter = warp & 3;
    const int lane_in_tile = quarter * 32 + lane;  // TMEM lane = A row of this CTA
    const int epilogue_thread = static_cast<int>(threadIdx.x) - 64;
    const int n_out = args.n_out;
    const int numerics = args.numerics;
    const float limit = args.swiglu_limit;
    uint32_t* const dump = static_cast<uint32_t*>(args.dump_acc);
    const bool up_half = kGateUp && lane_in_tile >= 64;
    int local = 0;
    for (int64_t unit = first_unit; unit < units; unit += unit_stride, ++local) {
      const int buffer = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      int item, block;
      decode_unit(args.items, unit, n_blocks, &item, &block);
      const int c0 = block * kChannelsPerUnit;
      const int expert = args.items[4 * item + 0];
      const int row0 = args.items[4 * item + 1];
      const int rows = args.items[4 * item + 2];
      // Output channel this thread finishes.
      const int n = kGateUp ? c0 + 64 * static_cast<int>(cta) + (lane_in_tile & 63) : c0 + kRowsPerCta * static_cast<int>(cta) + lane_in_tile;
      const bool channel_ok = n < n_out;
      ColumnMeta* meta = &ctl->meta[local & 1];
      for (int c = epilogue_thread; c < rows; c += 128) {
        if (kInt8) meta->scale[c] = args.a_scale[row0 + c];
        meta->target[c] = (kGateUp || kDense) ? row0 + c : args.sorted_routes[row0 + c];
      }
      float scale_gate = 1.0f, scale_up = 1.0f;
      if (kInt8 && channel_ok) {
        const float* s = args.w_scale + static_cast<int64_t>(expert) * n_total;
        scale_gate = s[n];
        if (kGateUp) scale_up = s[n + n_out];
      }
      float bias = 0.0f;
      if (kDense && channel_ok && args.bias != nullptr) bias = args.bias[n];
      epilogue_bar_sync();  // metadata visible to the four epilogue warps
      ptx::mbar_wait(&ctl->acc_full[buffer], use & 1u, abort_flag, status, 14);
      ptx::tcgen05_fence_after();
      const uint32_t acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buffer * kAccColumns);
      for (int col0 = 0; col0 < rows; col0 += 8) {
        uint32_t bits[8];
        ptx::tmem_ld_x8(acc + col0, bits);
        ptx::tmem_ld_wait();
        if constexpr (kGateUp) {
          // Gate threads finish columns 0..3 of the chunk, up threads columns 4..7; each sends the other half.
          const int channel = lane_in_tile & 63;
          uint32_t* send = ctl->exchange[up_half ? 1 : 0][channel];
#pragma unroll
          for (int j = 0; j < 4; ++j) send[j] = bits[up_half ? j : 4 + j];
          epilogue_bar_sync();
          const uint32_t* receive = ctl->exchange[up_half ? 0 : 1][channel];
          uint32_t other[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) other[j] = receive[j];
          epilogue_bar_sync();
          if (channel_ok) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int column = col0 + (up_half ? 4 + j : j);
              if (column < rows) {
                const int64_t row = meta->target[column];
                const uint32_t gate_bits = up_half ? other[j] : bits[j];
                const uint32_t up_bits = up_half ? bits[4 + j] : other[j];
                if (dump != nullptr) {
                  uint32_t* out = dump + row * n_total;
                  out[n] = gate_bits;
                  out[n + n_out] = up_bits;
                }
                float gate, up;
                if constexpr (kInt8) {
                  const float a = meta->scale[column];
                  gate = dequantize(static_cast<int>(gate_bits), a, scale_gate, numerics);
                  up = dequantize(static_cast<int>(up_bits), a, scale_up, numerics);
                } else {
                  gate = __uint_as_float(gate_bits);
                  up = __uint_as_float(up_bits);
                }
                args.y[row * n_out + n] = swiglu_to_bf16(gate, up, limit);
              }
            }
          }
        } else if (channel_ok) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (col0 + j < rows) {
              const int64_t target = meta->target[col0 + j];
              if (dump != nullptr) dump[static_cast<int64_t>(row0 + col0 + j) * n_total + n] = bits[j];
              float value;
              if constexpr (kInt8) {
                value = dequantize(static_cast<int>(bits[j]), meta->scale[col0 + j], scale_gate, numerics);
              } else {
                value = __uint_as_float(bits[j]);
              }
              if constexpr (kDense) {
                value = __fadd_rn(value, bias);
                if (args.dense_out_bf16) {
                  static_cast<uint16_t*>(args.dense_out)[target * n_out + n] = f32_to_bf16_bits(value);
                } else {
                  static_cast<float*>(args.dense_out)[target * n_out + n] = value;
                }
              } else {
                args.route_out[target * n_out + n] = value;
              }
            }
          }
        }
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(ptx::smem_u32(&ctl->acc_empty[buffer]), 0));
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  cluster_sync();  // neither CTA leaves while its peer may still signal its barriers or read its operands
  if (warp == 1) {
    __syncwarp();
    ptx::tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemColumns);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* symbol = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &query) == cudaSuccess &&
        query == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(symbol);
    }
  }
  return fn;
}

bool make_tensor_map(CUtensorMap* map, const void* base, bool int8, uint64_t rows, uint64_t k, uint32_t box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const uint32_t elem_bytes = int8 ? 1 : 2;
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {k * elem_bytes};
  const cuuint32_t box[2] = {kBlockKBytes / elem_bytes, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  return encode(map, int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool kInt8, bool kGateUp, bool kDense>
cudaError_t launch_pair(const GroupedGemmArgs& args, cudaStream_t stream) {
  auto kernel = umma_pair_grouped_gemm_kernel<kInt8, kGateUp, kDense>;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes));
    if (err != cudaSuccess) return err;
    configured = true;
  }
  const int n_total = kGateUp ? 2 * args.n_out : args.n_out;
  CUtensorMap weight_map, token_map;
  if (!make_tensor_map(&weight_map, args.weights, kInt8, static_cast<uint64_t>(args.experts) * n_total, args.k, kGateUp ? 64 : kRowsPerCta) ||
      !make_tensor_map(&token_map, args.a_rows, kInt8, static_cast<uint64_t>(args.total_rows), args.k, kRowsPerCta)) {
    return cudaErrorInvalidValue;
  }
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int channels_per_unit = kGateUp ? 128 : 256;
  const int n_blocks = (args.n_out + channels_per_unit - 1) / channels_per_unit;
  int64_t pairs = static_cast<int64_t>(args.max_items) * n_blocks;
  if (pairs > sms / 2) pairs = sms / 2;
  if (pairs <= 0) return cudaSuccess;
  kernel<<<static_cast<unsigned>(2 * pairs), kThreads, kSmemBytes, stream>>>(weight_map, token_map, args);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_umma_pair_grouped_gemm(const GroupedGemmArgs& args, bool int8, bool gate_up, cudaStream_t stream) {
  if (args.max_items <= 0 || args.total_rows <= 0) return cudaSuccess;
  if (args.dense_out != nullptr) {
    if (!int8 || gate_up) return cudaErrorInvalidValue;
    return launch_pair<true, false, true>(args, stream);
  }
  if (int8) return gate_up ? launch_pair<true, true, false>(args, stream) : launch_pair<true, false, false>(args, stream);
  return gate_up ? launch_pair<false, true, false>(args, stream) : launch_pair<false, false, false>(args, stream);
}

}  // namespace fmoe
