// Grouped expert GEMM, two-SM form: a cluster of two CTAs drives `tcgen05.mma.cta_group::2` so that a
// 256 (channels) x 256 (tokens) tile costs each SM only 128 + 128 operand rows per K step.
//
// Same work as umma_gemm.cu (the reference's two run_stage sweeps and their epilogues,
// csrc/moe/arm/i8mm_w8a8/kernels.cpp:328-368, 230-257) for the prefill regime, where an expert has
// hundreds of rows.  Three things bound that regime and shape this kernel:
//   * one thread issues every MMA, and a dependent instruction costs it several clocks: a 128 x 128 x 32-byte
//     MMA runs 66 clocks, so anything beyond a dozen instructions per MMA starves the tensor pipe.  The pair
//     issues 256 x 256 MMAs (132 clocks each) from a loop that only adds constants to descriptor words;
//   * a 128 x 128 tile reads 8 KB of shared memory per 66 clocks, the full shared-memory bandwidth; here
//     each SM reads 4 + 4 KB per 132 clocks;
//   * the epilogue handles 128 x 256 accumulators per CTA per unit: eight warps, 32-column tensor-memory
//     loads, per-column metadata fetched one unit ahead, no block-wide barrier inside a unit.
//
// Pair layout.  CTA r of the pair (r = 0 leads) stages its own halves: 128 A rows (weight channels)
// and 128 B rows (tokens); the MMA reads A rows 0..127 from CTA 0 and 128..255 from CTA 1, B likewise,
// and leaves D rows 128r..128r+127 x 256 token columns in CTA r's tensor memory.
//   down:    A rows of CTA r = channels n0 + 128 r .. + 127.
//   gate_up: A rows of CTA r = channels c0 + 64 r .. + 63 as four groups of [16 gate rows | 16 up rows]
//            (one 5-D TMA box: {K bytes, 16 rows, gate/up, 4 groups, expert}), so lanes l and l + 16 of every
//            epilogue warp hold gate and up of the same channel and swap them with one shuffle.
// Barriers.  Both producers signal the leader's "full" barrier (TMA complete_tx through the cluster
// address), the leader's single MMA thread commits to the "empty" and "accumulator full" barriers of
// both CTAs, and the follower's epilogue warps arrive on the leader's "accumulator empty" barrier
// through its cluster address.  No load is a multicast load.  Every wait is bounded (see ptx.cuh).
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace fmoe {

namespace {

constexpr int kRowsPerCta = 128;    // A rows and B rows staged by one CTA
constexpr int kPairTokens = 256;    // MMA N
constexpr int kBlockKBytes = 128;
constexpr int kUmmaKBytes = 32;
#ifndef FMOE_PAIR_EPILOGUE_WARPS
#define FMOE_PAIR_EPILOGUE_WARPS 8
#endif
constexpr int kEpilogueWarps = FMOE_PAIR_EPILOGUE_WARPS;  // a multiple of 4: every TMEM lane quarter gets the same number
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kThreads = 64 + kEpilogueThreads;
constexpr int kStages = 6;
constexpr int kStageBytes = 2 * kRowsPerCta * kBlockKBytes;  // 32 KB
constexpr int kAccColumns = kPairTokens;                     // one accumulator: 256 columns
constexpr int kTmemColumns = 512;                            // two accumulators
constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kStageBytes + 8192;

// Per-column values of a work unit, staged one unit ahead so that the element loop reads shared memory.
struct ColumnMeta {
  float scale[256];      // activation scale of the row (int8)
  uint64_t rowptr[256];  // byte address of the output row (down / dense; may be peer memory)
};

struct PairControl {
  ColumnMeta meta[2];  // first: its arrays are read with 16-byte loads
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  uint32_t exp_table[64];  // copy of kExp2Table: divergent lookups are served by 32 banks
};
static_assert(sizeof(PairControl) <= 8192, "control block exceeds its shared-memory reservation");

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

// TMA tiled loads whose completion bytes go to an mbarrier given by its cluster address (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar_cluster_address, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_address), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_5d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar_cluster_address, int c0, int c1,
                                                 int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_address), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
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

// D[tmem] (+)= A * B with the descriptors given as their 32-bit halves: the high word is the same for every
// operand tile of this kernel and the low word only ever has constants added to it, so the issuing thread
// spends one integer add per operand per MMA.
template <bool kInt8>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                          uint32_t accumulate) {
  if constexpr (kInt8) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %4, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld_x32(uint32_t address, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, "
      "%19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
        "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(address)
      : "memory");
}

__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory"); }

// Work unit -> (work item, channel block), item-major: the units of one item (same token rows, successive
// channel blocks) are adjacent, and the same channel block of the next row tile of an expert is n_blocks
// units further, i.e. in flight on another pair at about the same time, so its weight tile comes from L2.
struct TrueTag {
  static constexpr bool value = true;
};
struct FalseTag {
  static constexpr bool value = false;
};

struct UnitInfo {
  int expert, row0, rows, block;
};

// rows_per_route: 2 in the two-plane form (first row and row count come back in token rows), else 1.
__device__ __forceinline__ UnitInfo load_unit(const int* __restrict__ items, int64_t unit, int64_t units, int n_blocks, int rows_per_route = 1) {
  UnitInfo info = {0, 0, 0, 0};
  if (unit < units) {
    const int item = static_cast<int>(unit / n_blocks);
    const int4 packed = __ldg(reinterpret_cast<const int4*>(items) + item);
    info.expert = packed.x;
    info.row0 = packed.y * rows_per_route;
    info.rows = packed.z * rows_per_route;
    info.block = static_cast<int>(unit - static_cast<int64_t>(item) * n_blocks);
  }
  return info;
}

// The same unit with every field taken from lane 0 (all lanes hold the same values already).
__device__ __forceinline__ UnitInfo warp_uniform(UnitInfo info) {
  info.expert = __shfl_sync(0xffffffffu, info.expert, 0);
  info.row0 = __shfl_sync(0xffffffffu, info.row0, 0);
  info.rows = __shfl_sync(0xffffffffu, info.rows, 0);
  info.block = __shfl_sync(0xffffffffu, info.block, 0);
  return info;
}

// kPlanes (an instance of the int8 kernel; W8A16 in its fixed-point form): every route arrives as two int8 token rows,
// the high plane at row 2p and the low plane at row 2p + 1 of its 16-bit fixed-point activations, so a work item of r
// routes has 2r token rows (at most 128 routes) and accumulator columns (2j, 2j + 1) belong to route j: the exact
// integer dot product is 256 * column(2j) + column(2j + 1) (common.cuh: dequantize_planes).  Work items are given in
// routes; loads, the MMA's N and the epilogue count plane rows.
template <bool kInt8, bool kGateUp, bool kDense, bool kPlanes = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
umma_pair_grouped_gemm_kernel(const __grid_constant__ CUtensorMap weight_map, const __grid_constant__ CUtensorMap token_map,
                              GroupedGemmArgs args) {
  static_assert(!kPlanes || (kInt8 && !kDense), "the two-plane form is an instance of the int8 grouped kernel");
  constexpr int kElemBytes = kInt8 ? 1 : 2;
  constexpr int kBlockKElems = kBlockKBytes / kElemBytes;
  constexpr int kChannelsPerUnit = kGateUp ? 128 : 256;  // output channels one pair finishes per work unit
  constexpr int kRowsPerRoute = kPlanes ? 2 : 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  PairControl* ctl = reinterpret_cast<PairControl*>(smem + static_cast<size_t>(kStages) * kStageBytes);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);  // the same value, known to be warp-uniform
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_cta_rank();
  const bool leader = cta == 0;
  int* status = args.status_rw;

  // (Values that come from global loads pass through a shuffle where the warps that feed TMA and the tensor pipe use
  // them: it changes nothing but lets the compiler treat them as warp-uniform.)
  const int items = __shfl_sync(0xffffffffu, min(args.status[args.item_count_word], args.max_items), 0);
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
      ptx::mbar_init(&ctl->acc_empty[b], 2 * kEpilogueWarps);  // the epilogue warps of both CTAs
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
  }
  if (threadIdx.x >= 64 && threadIdx.x < 128) ctl->exp_table[threadIdx.x - 64] = kExp2Table[threadIdx.x - 64];
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, kTmemColumns);
    tmem_relinquish_pair();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  cluster_sync();  // the peer's barriers are initialised before anything signals them
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, ctl->tmem_base, 0);
  volatile int* abort_flag = &ctl->abort_flag;
  const uint32_t smem_base = ptx::smem_u32(smem);

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    // The whole warp walks the loop; one elected lane issues the loads (ptx::elect_one).
    {
      const bool issuer = ptx::elect_one();
      if (issuer) {
        ptx::prefetch_tensormap(&weight_map);
        ptx::prefetch_tensormap(&token_map);
      }
      const uint32_t full_leader0 = map_to_cta(ptx::smem_u32(&ctl->full[0]), 0);
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      UnitInfo cur = warp_uniform(load_unit(args.items, first_unit, units, n_blocks, kRowsPerRoute));
      for (int64_t unit = first_unit; unit < units; unit += unit_stride) {
        const UnitInfo next = warp_uniform(load_unit(args.items, unit + unit_stride, units, n_blocks, kRowsPerRoute));  // in flight during this unit
        // The MMA takes the first N/2 token rows from the leader's tile and the other N/2 from the follower's.
        const int mma_n = min(kPairTokens, (cur.rows + 31) & ~31);
        const int token_row = cur.row0 + (mma_n / 2) * static_cast<int>(cta);
        const int channel0 = cur.block * kChannelsPerUnit + (kChannelsPerUnit / 2) * static_cast<int>(cta);
        const int weight_row = cur.expert * n_total + channel0;  // down
        const int group = channel0 >> 4;                         // gate_up: 16-channel group
        for (int kb = 0; kb < k_blocks; ++kb) {
          ptx::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag, status, 11);
          if (!issuer) {
            // the other lanes only keep step
          } else if (FMOE_DIAG_BIT(args, 2)) {
            if (leader) ptx::mbar_arrive(&ctl->full[stage]);
          } else {
            const uint32_t dst = smem_base + static_cast<uint32_t>(stage) * kStageBytes;
            const uint32_t bar = full_leader0 + 8u * static_cast<uint32_t>(stage);
            if (leader) ptx::mbar_arrive_expect_tx(&ctl->full[stage], 2 * kStageBytes);
            const int x = kb * kBlockKElems;
            if constexpr (kGateUp) {
              if (args.gate_up_one_box) {
                // One 16 KB box of four groups of [16 gate rows | 16 up rows]: tensor dimensions
                // {K, row in group, gate/up, group, expert}.
                tma_load_5d_pair(dst, &weight_map, bar, x, 0, 0, group, cur.expert);
              } else {
                // The same rows as four 4 KB boxes: tensor dimensions {K, row in group, group, gate/up, expert}.
#pragma unroll
                for (int g = 0; g < 4; ++g) tma_load_5d_pair(dst + g * 32 * kBlockKBytes, &weight_map, bar, x, 0, group + g, 0, cur.expert);
              }
            } else {
              tma_load_2d_pair(dst, &weight_map, bar, x, weight_row);
            }
            tma_load_2d_pair(dst + kRowsPerCta * kBlockKBytes, &token_map, bar, x, token_row);
          }
          ++issued;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        cur = next;
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
    // The whole warp walks the loop (waits included); one elected lane issues the MMAs and commits (ptx::elect_one).
    if (leader) {
      const bool issuer = ptx::elect_one();
      // Descriptor words (see ptx::make_smem_desc_sw128): the low word holds the start address >> 4 and the
      // ignored leading offset, the high word the 1024-byte group stride, version 1 and SWIZZLE_128B.
      const uint32_t desc_hi = static_cast<uint32_t>(1024 >> 4) | (1u << 14) | (2u << 29);
      const uint32_t a_lo_stage0 = ((smem_base & 0x3ffffu) >> 4) | (1u << 16);
      constexpr uint32_t kStageStep = kStageBytes >> 4;
      constexpr uint32_t kTokenStep = (kRowsPerCta * kBlockKBytes) >> 4;
      const uint32_t empty_c0 = map_to_cta(ptx::smem_u32(&ctl->empty[0]), 0);
      const uint32_t empty_c1 = map_to_cta(ptx::smem_u32(&ctl->empty[0]), 1);
      const uint32_t accfull_c0 = map_to_cta(ptx::smem_u32(&ctl->acc_full[0]), 0);
      const uint32_t accfull_c1 = map_to_cta(ptx::smem_u32(&ctl->acc_full[0]), 1);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t a_lo = a_lo_stage0;
      int local = 0;
      UnitInfo cur = load_unit(args.items, first_unit, units, n_blocks, kRowsPerRoute);
      for (int64_t unit = first_unit; unit < units; unit += unit_stride, ++local) {
        const UnitInfo next = load_unit(args.items, unit + unit_stride, units, n_blocks, kRowsPerRoute);
        const uint32_t buffer = static_cast<uint32_t>(local) & 1u;
        const uint32_t use = static_cast<uint32_t>(local) >> 1;
        // N follows the rows this unit really has (a multiple of 32 for two-SM MMAs).  The row count comes from a global
        // load; the shuffle tells the compiler that every lane holds the same value.
        const int unit_rows = __shfl_sync(0xffffffffu, cur.rows, 0);
        const int mma_n = min(kPairTokens, (unit_rows + 31) & ~31);
        const uint32_t idesc = ptx::make_instr_desc(kInt8, 2 * kRowsPerCta, mma_n);
        ptx::mbar_wait(&ctl->acc_empty[buffer], (use & 1u) ^ 1u, abort_flag, status, 12);
        ptx::tcgen05_fence_after();
        const uint32_t acc = tmem_base + buffer * kAccColumns;
        uint32_t accumulate = 0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ptx::mbar_wait(&ctl->full[stage], phase, abort_flag, status, 13);
          ptx::tcgen05_fence_after();
          if (issuer) {
            if (!FMOE_DIAG_BIT(args, 4)) {
#pragma unroll
              for (uint32_t ks = 0; ks < kBlockKBytes / kUmmaKBytes; ++ks) {
                umma_pair<kInt8>(acc, a_lo + 2u * ks, a_lo + kTokenStep + 2u * ks, desc_hi, idesc, ks == 0 ? accumulate : 1u);
              }
            }
            tcgen05_commit_pair(empty_c0 + 8u * static_cast<uint32_t>(stage));
            tcgen05_commit_pair(empty_c1 + 8u * static_cast<uint32_t>(stage));
          }
          accumulate = 1;
          a_lo += kStageStep;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
            a_lo = a_lo_stage0;
          }
        }
        if (issuer) {
          tcgen05_commit_pair(accfull_c0 + 8u * buffer);
          tcgen05_commit_pair(accfull_c1 + 8u * buffer);
        }
        cur = next;
      }
    }
  } else {
    // ---------------- epilogue (warps 2.. of both CTAs) ----------------
    const int quarter = warp & 3;                    // the TMEM lanes a warp may read are fixed by warp id % 4
    const int chunk_first = (warp - 2) >> 2;         // warps sharing a lane quarter take 32-column chunks round-robin
    constexpr int kChunkStep = kEpilogueWarps / 4;
    const int lane_in_tile = quarter * 32 + lane;    // TMEM lane = A row of this CTA
    const int tid = static_cast<int>(threadIdx.x) - 64;  // threads 0..255 each stage the metadata of one column
    const int n_out = args.n_out;
    const bool native = args.numerics == FMOE_NUMERICS_NATIVE;
    const float limit = args.swiglu_limit;
    const int activation = args.activation;
    uint32_t* const dump = kPlanes ? nullptr : static_cast<uint32_t*>(args.dump_acc);  // the dump holds one row per route
    const bool low = lane < 16;  // gate_up: lanes 0..15 hold gate rows, lanes 16..31 the up rows of the same channels
    // Output channel of this thread inside the unit's channel block.
    const int channel_in_unit = kGateUp ? 64 * static_cast<int>(cta) + 16 * quarter + (lane & 15)
                                        : kRowsPerCta * static_cast<int>(cta) + lane_in_tile;
    const uint32_t acc_empty_leader = map_to_cta(ptx::smem_u32(&ctl->acc_empty[0]), 0);
    const uint32_t acc_lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t* exp_table = ctl->exp_table;

    // Per-unit values: the column metadata in shared memory and this thread's weight scales in registers.  Both
    // are fetched while the previous unit is being finished.
    struct ThreadUnit {
      float column_scale;      // of column `tid`
      uint64_t column_rowptr;  // of column `tid`: byte address of its output row (down / dense)
      float scale_gate, scale_up, bias;
    };
    auto fetch = [&](const UnitInfo& info, bool valid) {
      ThreadUnit t = {0.0f, 0ull, kInt8 ? 1.0f : 0.0f, kInt8 ? 1.0f : 0.0f, 0.0f};
      if (!valid) return t;
      if (tid < info.rows) {
        const int row = (info.row0 + tid) / kRowsPerRoute;  // sorted position of the column's route
        if (kInt8) t.column_scale = args.a_scale[row];
        if constexpr (kDense) {
          t.column_rowptr = reinterpret_cast<uint64_t>(args.dense_out) + static_cast<uint64_t>(row) * n_out * (args.dense_out_bf16 ? 2 : 4);
        } else if constexpr (!kGateUp) {
          t.column_rowptr = args.row_out_ptrs != nullptr
                                ? args.row_out_ptrs[row]
                                : reinterpret_cast<uint64_t>(args.route_out) +
                                      static_cast<uint64_t>(args.sorted_routes[row]) * n_out * (args.route_out_bf16 ? 2 : 4);
        }
      }
      const int n = info.block * kChannelsPerUnit + channel_in_unit;
      if (n < n_out) {
        if (kInt8) {
          const float* s = args.w_scale + static_cast<int64_t>(info.expert) * n_total;
          t.scale_gate = s[n];
          if (kGateUp) t.scale_up = s[n + n_out];
        }
        if (kDense && args.bias != nullptr) t.bias = args.bias[n];
        if (!kInt8 && !kDense && args.expert_bias != nullptr) {
          // BF16 path: the per-expert bias rides in the scale slots (unused without int8) and is ADDED.
          const float* b = args.expert_bias + static_cast<int64_t>(info.expert) * n_total;
          t.scale_gate = b[n];
          if (kGateUp) t.scale_up = b[n + n_out];
        }
      }
      return t;
    };

    // One accumulator value -> fp32 (int8: the reference's two multiplication orders, chosen at compile time).
    auto to_float = [&](auto native_tag, uint32_t bits, float a, float s) {
      if constexpr (kInt8) {
        const float value = static_cast<float>(static_cast<int>(bits));
        if constexpr (decltype(native_tag)::value) {
          return __fmul_rn(value, __fmul_rn(a, s));
        } else {
          return __fmul_rn(__fmul_rn(value, a), s);
        }
      } else {
        return __fadd_rn(__uint_as_float(bits), s);  // s = the channel's bias (0 without one)
      }
    };
    // Calls body(fast, native) with both flags turned into types: four instances of the element loop, one branch.
    auto dispatch = [&](bool fast, auto&& body) {
      if (fast) {
        if (native) {
          body(TrueTag{}, TrueTag{});
        } else {
          body(TrueTag{}, FalseTag{});
        }
      } else {
        if (native) {
          body(FalseTag{}, TrueTag{});
        } else {
          body(FalseTag{}, FalseTag{});
        }
      }
    };

    UnitInfo cur = load_unit(args.items, first_unit, units, n_blocks, kRowsPerRoute);
    UnitInfo next = load_unit(args.items, first_unit + unit_stride, units, n_blocks, kRowsPerRoute);
    ThreadUnit mine = fetch(cur, first_unit < units);
    if (tid < 256) {
      ctl->meta[0].scale[tid] = mine.column_scale;
      ctl->meta[0].rowptr[tid] = mine.column_rowptr;
    }
    epilogue_bar_sync();

    int local = 0;
    for (int64_t unit = first_unit; unit < units; unit += unit_stride, ++local) {
      const uint32_t buffer = static_cast<uint32_t>(local) & 1u;
      const uint32_t use = static_cast<uint32_t>(local) >> 1;
      // Loads for the next unit (and the work item of the one after) are issued now and consumed after this unit.
      const ThreadUnit upcoming = fetch(next, unit + unit_stride < units);
      const UnitInfo after = load_unit(args.items, unit + 2 * unit_stride, units, n_blocks, kRowsPerRoute);

      const int rows = cur.rows;
      const int row0 = cur.row0;
      const int n = cur.block * kChannelsPerUnit + channel_in_unit;
      const bool channel_ok = n < n_out;
      const bool block_full = (cur.block + 1) * kChannelsPerUnit <= n_out;  // every thread's channel exists
      const ColumnMeta* meta = &ctl->meta[local & 1];
      const int chunks = FMOE_DIAG_BIT(args, 1) ? 0 : (rows + 31) >> 5;

      ptx::mbar_wait(&ctl->acc_full[buffer], use & 1u, abort_flag, status, 14);
      ptx::tcgen05_fence_after();
      const uint32_t acc = acc_lane_base + buffer * kAccColumns;
      for (int chunk = chunk_first; chunk < chunks; chunk += kChunkStep) {
        uint32_t v[32];
        tmem_ld_x32(acc + static_cast<uint32_t>(chunk * 32), v);
        ptx::tmem_ld_wait();
        const int col0 = chunk * 32;
        const bool fast = block_full && col0 + 32 <= rows && dump == nullptr;  // warp-uniform
        if constexpr (kGateUp && kPlanes) {
          // Columns 4q .. 4q + 3 are the (high, low) planes of two routes.  Lanes l (gate) and l + 16 (up) hold the same
          // channel: the gate lane finishes the first route of the four columns, the up lane the second, each receiving
          // the other's two plane values of that route.
          const float* scale = meta->scale + col0;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t first = __shfl_xor_sync(0xffffffffu, low ? v[4 * q + 2] : v[4 * q], 16);
            const uint32_t second = __shfl_xor_sync(0xffffffffu, low ? v[4 * q + 3] : v[4 * q + 1], 16);
            const int column = col0 + 4 * q + (low ? 0 : 2);  // plane row of this lane's route inside the item
            if (column >= rows || !channel_ok) continue;
            const int gate_high = static_cast<int>(low ? v[4 * q] : first);
            const int gate_low = static_cast<int>(low ? v[4 * q + 1] : second);
            const int up_high = static_cast<int>(low ? first : v[4 * q + 2]);
            const int up_low = static_cast<int>(low ? second : v[4 * q + 3]);
            const float a = scale[4 * q + (low ? 0 : 2)];
            const float gate = dequantize_planes(gate_high, gate_low, a, mine.scale_gate);
            const float up = dequantize_planes(up_high, up_low, a, mine.scale_up);
            args.y[static_cast<int64_t>((row0 + column) >> 1) * n_out + n] =
                activation == FMOE_ACT_SILU ? swiglu_to_bf16_with(gate, up, limit, exp_table) : other_activation_to_bf16(activation, gate, up);
          }
        } else if constexpr (kPlanes) {
          // down: adjacent columns are the two planes of one route; the route's output row address is staged per column.
          const bool bf16_out = args.route_out_bf16 != 0;
          const uint64_t n_bytes = static_cast<uint64_t>(n) * (bf16_out ? 2 : 4);
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const int column = col0 + j;
            if (column >= rows || !channel_ok) continue;
            const float value = dequantize_planes(static_cast<int>(v[j]), static_cast<int>(v[j + 1]), meta->scale[column], mine.scale_gate);
            const uint64_t rowptr = meta->rowptr[column];
            if (bf16_out) {
              *reinterpret_cast<uint16_t*>(rowptr + n_bytes) = f32_to_bf16_bits(value);
            } else {
              *reinterpret_cast<float*>(rowptr + n_bytes) = value;
            }
          }
        } else if constexpr (kGateUp) {
          // Lanes l (gate) and l + 16 (up) hold the same channel: the gate lane finishes the even columns, the
          // up lane the odd ones, each receiving the other's value of that column.  Output rows are the sorted
          // rows themselves: row0 + column.
          uint16_t* const out0 = args.y + (static_cast<int64_t>(row0 + col0 + (low ? 0 : 1)) * n_out + n);
          const uint32_t pair_stride = 2u * static_cast<uint32_t>(n_out);
          const float4* scale4 = reinterpret_cast<const float4*>(meta->scale + col0);
          auto body = [&](auto fast_tag, auto native_tag) {
            constexpr bool kFast = decltype(fast_tag)::value;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 s4 = scale4[q];  // the scales of columns 4q .. 4q+3 (one broadcast load)
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int p = 2 * q + h;
                const uint32_t received = __shfl_xor_sync(0xffffffffu, low ? v[2 * p + 1] : v[2 * p], 16);
                const uint32_t gate_bits = low ? v[2 * p] : received;
                const uint32_t up_bits = low ? received : v[2 * p + 1];
                const float a = h == 0 ? (low ? s4.x : s4.y) : (low ? s4.z : s4.w);
                if constexpr (!kFast) {
                  const int column = col0 + 2 * p + (low ? 0 : 1);
                  if (column >= rows || !channel_ok) continue;
                  if (dump != nullptr) {
                    uint32_t* out = dump + static_cast<int64_t>(row0 + column) * n_total;
                    out[n] = gate_bits;
                    out[n + n_out] = up_bits;
                  }
                }
                const float gate = to_float(native_tag, gate_bits, a, mine.scale_gate);
                const float up = to_float(native_tag, up_bits, a, mine.scale_up);
                out0[static_cast<uint32_t>(p) * pair_stride] =
                    (kInt8 || activation == FMOE_ACT_SILU) ? swiglu_to_bf16_with(gate, up, limit, exp_table)
                                                           : other_activation_to_bf16(activation, gate, up);
              }
            }
          };
          dispatch(fast, body);
        } else {
          const float4* scale4 = reinterpret_cast<const float4*>(meta->scale + col0);
          const ulonglong2* rowptr2 = reinterpret_cast<const ulonglong2*>(meta->rowptr + col0);
          const bool bf16_out = kDense ? args.dense_out_bf16 != 0 : args.route_out_bf16 != 0;
          const uint64_t n_bytes = static_cast<uint64_t>(n) * (bf16_out ? 2 : 4);
          auto body = [&](auto fast_tag, auto native_tag) {
            constexpr bool kFast = decltype(fast_tag)::value;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 s4 = scale4[q];
              const ulonglong2 p01 = rowptr2[2 * q];
              const ulonglong2 p23 = rowptr2[2 * q + 1];
              const float scales[4] = {s4.x, s4.y, s4.z, s4.w};
              const uint64_t rowptrs[4] = {p01.x, p01.y, p23.x, p23.y};
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                const int j = 4 * q + h;
                if constexpr (!kFast) {
                  const int column = col0 + j;
                  if (column >= rows || !channel_ok) continue;
                  if (dump != nullptr) dump[static_cast<int64_t>(row0 + column) * n_total + n] = v[j];
                }
                float value = to_float(native_tag, v[j], scales[h], mine.scale_gate);
                if constexpr (kDense) {
                  value = __fadd_rn(value, mine.bias);
                  if (bf16_out) {
                    *reinterpret_cast<uint16_t*>(rowptrs[h] + n_bytes) = f32_to_bf16_bits(value);
                  } else {
                    *reinterpret_cast<float*>(rowptrs[h] + n_bytes) = value;
                  }
                } else if (bf16_out) {
                  *reinterpret_cast<uint16_t*>(rowptrs[h] + n_bytes) = f32_to_bf16_bits(value);
                } else {
                  *reinterpret_cast<float*>(rowptrs[h] + n_bytes) = value;
                }
              }
            }
          };
          dispatch(fast, body);
        }
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader + 8u * buffer);

      // Publish the next unit's column metadata.  Nobody still reads that buffer: it belonged to the previous
      // unit, which every warp left before the barrier at the end of the previous iteration.
      if (tid < 256) {
        ColumnMeta* meta_next = &ctl->meta[(local + 1) & 1];
        meta_next->scale[tid] = upcoming.column_scale;
        meta_next->rowptr[tid] = upcoming.column_rowptr;
      }
      epilogue_bar_sync();
      mine = upcoming;
      cur = next;
      next = after;
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

// 2-D K-major tensor [rows, k] with 128-byte-swizzled boxes of {128 bytes of K, box_rows}.
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

// gate_up weights [E, 2I, K] as a 5-D tensor whose boxes put the 16 gate rows of a channel group next to its 16
// up rows.  one_box: dimensions {K, 16 rows, gate|up, I/16 groups, E} and a box of four groups (16 KB, one TMA
// operation per stage; the gate|up stride is larger than the group stride that follows it).  Otherwise
// {K, 16 rows, I/16 groups, gate|up, E} with strides in ascending order and a box of one group (4 KB, four
// operations per stage): the fallback if the driver refuses the first encoding.
bool make_gate_up_map(CUtensorMap* map, const void* base, bool int8, uint64_t experts, uint64_t inter, uint64_t k, bool one_box) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const uint64_t elem_bytes = int8 ? 1 : 2;
  const uint64_t row_bytes = k * elem_bytes;
  const cuuint32_t inner = static_cast<cuuint32_t>(kBlockKBytes / elem_bytes);
  const cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType type = int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (one_box) {
    const cuuint64_t dims[5] = {k, 16, 2, inter / 16, experts};
    const cuuint64_t strides[4] = {row_bytes, inter * row_bytes, 16 * row_bytes, 2 * inter * row_bytes};
    const cuuint32_t box[5] = {inner, 16, 2, 4, 1};
    return encode(map, type, 5, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const cuuint64_t dims[5] = {k, 16, inter / 16, 2, experts};
  const cuuint64_t strides[4] = {row_bytes, 16 * row_bytes, inter * row_bytes, 2 * inter * row_bytes};
  const cuuint32_t box[5] = {inner, 16, 1, 2, 1};
  return encode(map, type, 5, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool kInt8, bool kGateUp, bool kDense, bool kPlanes = false>
cudaError_t launch_pair(const GroupedGemmArgs& args, cudaStream_t stream) {
  auto kernel = umma_pair_grouped_gemm_kernel<kInt8, kGateUp, kDense, kPlanes>;
  static PerDeviceOnce configured;
  const int device = current_device_ordinal();
  if (configured.needed(device)) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes));
    if (err != cudaSuccess) return err;
    configured.mark(device);
  }
  const int n_total = kGateUp ? 2 * args.n_out : args.n_out;
  CUtensorMap weight_map, token_map;
  GroupedGemmArgs launch_args = args;
  bool weights_ok;
  if (kGateUp) {
    bool try_one = args.n_out % 64 == 0;
#ifdef FMOE_DIAG
    const char* forced = getenv("FUSED_CPP_MOE_GATE_UP_BOXES");  // diagnostic library only: "4" forces the four-box encoding
    if (forced != nullptr && forced[0] == '4') try_one = false;
#endif
    launch_args.gate_up_one_box = try_one && make_gate_up_map(&weight_map, args.weights, kInt8, args.experts, args.n_out, args.k, true);
    weights_ok = launch_args.gate_up_one_box || make_gate_up_map(&weight_map, args.weights, kInt8, args.experts, args.n_out, args.k, false);
  } else {
    weights_ok = make_tensor_map(&weight_map, args.weights, kInt8, static_cast<uint64_t>(args.experts) * n_total, args.k, kRowsPerCta);
  }
  const uint64_t token_rows = static_cast<uint64_t>(args.total_rows) * (kPlanes ? 2 : 1);
  if (!weights_ok || !make_tensor_map(&token_map, args.a_rows, kInt8, token_rows, args.k, kRowsPerCta)) {
    return cudaErrorInvalidValue;
  }
  const int sms = sm_count_of_current_device();
  const int channels_per_unit = kGateUp ? 128 : 256;
  const int n_blocks = (args.n_out + channels_per_unit - 1) / channels_per_unit;
  int64_t pairs = static_cast<int64_t>(args.max_items) * n_blocks;
  if (pairs > sms / 2) pairs = sms / 2;
  if (pairs <= 0) return cudaSuccess;
  kernel<<<static_cast<unsigned>(2 * pairs), kThreads, kSmemBytes, stream>>>(weight_map, token_map, launch_args);
  return cudaGetLastError();
}

}  // namespace

// gate_up stages 16-channel groups through its 5-D tensor map.
bool umma_pair_supported(bool gate_up, int n_out, int64_t output_rows) {
  (void)output_rows;
  return !gate_up || n_out % 16 == 0;
}

cudaError_t launch_umma_pair_grouped_gemm(const GroupedGemmArgs& args, bool int8, bool gate_up, cudaStream_t stream) {
  if (args.max_items <= 0 || args.total_rows <= 0) return cudaSuccess;
  if (!umma_pair_supported(gate_up, args.n_out, args.total_rows)) return cudaErrorInvalidValue;
  if (args.w8a16 == 2) {
    // W8A16 in its fixed-point form: int8 kernel, two token rows per route, work items of at most 128 routes.
    if (!int8 || args.dense_out != nullptr || args.a_scale == nullptr) return cudaErrorInvalidValue;
    return gate_up ? launch_pair<true, true, false, true>(args, stream) : launch_pair<true, false, false, true>(args, stream);
  }
  if (args.dense_out != nullptr) {
    if (!int8 || gate_up) return cudaErrorInvalidValue;
    return launch_pair<true, false, true>(args, stream);
  }
  if (int8) return gate_up ? launch_pair<true, true, false>(args, stream) : launch_pair<true, false, false>(args, stream);
  return gate_up ? launch_pair<false, true, false>(args, stream) : launch_pair<false, false, false>(args, stream);
}

}  // namespace fmoe
