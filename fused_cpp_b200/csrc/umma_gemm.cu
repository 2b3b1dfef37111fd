// Grouped expert GEMM on the sm_100a tensor cores (tcgen05.mma, accumulators in tensor memory,
// operands staged in shared memory by TMA tiled loads).
//
// It does the work of the reference's two `run_stage` sweeps and their epilogues:
//   gate_up: acc = Xq * W13[e]^T (int8 -> int32, or bf16 -> fp32), then dequant, clamp, SiLU(gate)*up,
//            bf16 store            (csrc/moe/arm/i8mm_w8a8/kernels.cpp:328-368, 230-246;
//                                   BF16: csrc/moe/arm/sve_bf16/packing.cpp:51-73)
//   down:    acc = Yq * W2[e]^T, then route_out[flat route] = f32(acc) * (a2 * s2)  -- the scatter to
//            the flat route id is the un-permute (csrc/moe/arm/i8mm_w8a8/kernels.cpp:248-257, 659-671)
//
// Orientation.  The weight tile is the MMA's A operand (M = 128 output channels) and the expert's
// token rows are the B operand (N = row tile, 16..256), both K-major exactly as they lie in HBM
// ([E, N, K] weights, [rows, K] activations).  Every weight byte is therefore read once per
// (expert, row tile) whatever the number of rows, which is what the weight-streaming (decode)
// regime needs, and the same kernel covers prefill with a 128/256-row tile.  The accumulator
// D[channel, token] lives in TMEM: one lane per output channel, one 32-bit column per token.
// gate_up issues two MMAs per K step (gate rows n and up rows I+n against the same token tile) so
// that each epilogue thread holds the gate and the up value of the same (token, channel).
//
// CTA = 6 warps, persistent over work units (work item x 128-channel block), round-robin:
//   warp 0      TMA producer: per K block of 128 bytes, one or two weight tiles + the token tile;
//   warp 1      allocates TMEM, issues tcgen05.mma (one thread), commits to the stage's "empty"
//               barrier and, per work unit, to the accumulator's "full" barrier;
//   warps 2..5  epilogue: tcgen05.ld their 32-lane TMEM quarter, apply the epilogue, store.
// W8A16 (int8 weights, bf16 activations; the reference's fused_moe_w8a16_* ops, csrc/moe/arm/common/
// fused_moe_bf16_tiled.cpp:4916-5000, 8740-8760): the weight tile arrives as int8 (half the HBM bytes of bf16) in a
// landing area of the stage, eight more warps (6..13) widen it to bf16 -- exact, |q| <= 128 -- into the 128-byte
// swizzled operand tile the kind::f16 MMA reads, and the epilogue multiplies by the per-output-channel scale in
// fp32.  This instance runs TOKEN-MAJOR: the token tile is the A operand (M = 128 lanes = token rows, of which the
// item's rows are real) and the widened weight tile the B operand (N = 256 = 128 gate + 128 up channels, or 128 for
// down), because a tcgen05.mma of M = 128 takes about the same time whatever its N: with the weights on the N side
// one instruction covers 256 x 16 weights instead of 128 x 16, and the tensor pipe keeps up with int8 weights
// arriving at HBM speed (weight-major it could not: eight MMAs per 16 KB of weights against a budget of five).
// An epilogue thread then owns a token row and stores eight channels at a time.
// Accumulators are double-buffered in TMEM when two buffers fit in 512 columns, so the epilogue of
// one unit overlaps the main loop of the next.  No load uses cluster multicast; weight-tile reuse
// between row tiles of one expert comes from L2 (adjacent work items run concurrently).
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace fmoe {

namespace {

constexpr int kBlockM = 128;        // output channels per MMA tile (TMEM lanes)
constexpr int kBlockKBytes = 128;   // bytes of K per pipeline stage = one 128-byte swizzle row
constexpr int kUmmaKBytes = 32;     // bytes of K per tcgen05.mma
constexpr int kThreads = 192;
constexpr int kEpilogueWarp0 = 2;
constexpr int kConvertWarp0 = 6;          // W8A16: warps 6.. widen the int8 weight tile to bf16
#ifndef FMOE_W8A16_CONVERT_WARPS
#define FMOE_W8A16_CONVERT_WARPS 8
#endif
#ifndef FMOE_W8A16_STAGES
#define FMOE_W8A16_STAGES 2
#endif
constexpr int kConvertWarps = FMOE_W8A16_CONVERT_WARPS;
constexpr int kThreadsW8A16 = kThreads + kConvertWarps * 32;
constexpr int kLandingRowBytes = 64;      // W8A16: one K block = 64 weights = 64 int8 bytes per channel row
constexpr int kSmemBudget = 216 * 1024;  // operand stages; with the control block and alignment slack 224 KB of the 227 KB a CTA may have

// W8A16: the most operand stages (up to `wanted`) that still leave three landing slots in the budget.
constexpr int w8a16_stages(int wanted, int stage_bytes, int landing_bytes, int budget) {
  int stages = wanted;
  while (stages > 2 && (budget - stages * stage_bytes) / landing_bytes < 3) --stages;
  return stages;
}

template <bool kGateUp, int kRowTile, bool kW8A16 = false>
struct TileConfig {
  static constexpr int kWeightTiles = kGateUp ? 2 : 1;
  static constexpr int kWeightBytes = kWeightTiles * kBlockM * kBlockKBytes;
  static constexpr int kTokenBytes = kRowTile * kBlockKBytes;
  // W8A16: what arrives from HBM per K block -- the token tile (MMA-ready) and the int8 weight tiles -- lands in a ring
  // of its own (kLandingSlots slots: [token tile | int8 weights]) that runs as far ahead of the MMAs as shared memory
  // allows, since those are the bytes in flight that have to cover the memory latency.  An operand stage then only
  // holds the widened bf16 weight tile; a few stages suffice (widen one while the MMAs read another).
  static constexpr int kStageBytes = kW8A16 ? kWeightBytes : kWeightBytes + kTokenBytes;
  static constexpr int kInt8TileBytes = kWeightTiles * kBlockM * kLandingRowBytes;
  // W8A16 runs token-major (see the kernel): the token tile is the MMA's A operand and the MMA always reads 128 rows
  // of it, so its region is 128 rows tall whatever the row tile (the TMA load fills the first kRowTile rows).
  static constexpr int kTokenRegionBytes = kW8A16 ? kBlockM * kBlockKBytes : kTokenBytes;
  static constexpr int kLandingBytes = kW8A16 ? kTokenRegionBytes + kInt8TileBytes : 0;
  static constexpr int kStagesRaw = kW8A16 ? w8a16_stages(FMOE_W8A16_STAGES, kStageBytes, kTokenRegionBytes + kInt8TileBytes, kSmemBudget)
                                            : kSmemBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kLandingSlotsRaw = kW8A16 ? (kSmemBudget - kStages * kStageBytes) / kLandingBytes : 0;
  static constexpr int kLandingSlots = kLandingSlotsRaw > 8 ? 8 : kLandingSlotsRaw;
  static constexpr int kLandingOffset = kStages * kStageBytes;  // the landing ring follows the operand stages
  // Accumulator columns: tokens (weight-major: one block of kRowTile columns per weight tile) or, token-major,
  // the channels of the unit (128 per weight tile).
  static constexpr int kAccColumns = kW8A16 ? kWeightTiles * kBlockM : kWeightTiles * kRowTile;
  static constexpr int kAccBuffers = (2 * kAccColumns <= 512) ? 2 : 1;
  static constexpr int kTmemColumnsRaw = kAccBuffers * kAccColumns;
  static constexpr int kTmemColumns = kTmemColumnsRaw <= 32 ? 32 : kTmemColumnsRaw <= 64 ? 64 : kTmemColumnsRaw <= 128 ? 128
                                      : kTmemColumnsRaw <= 256 ? 256 : 512;
  static constexpr int kOperandBytes = kStages * kStageBytes + kLandingSlots * kLandingBytes;
  static constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + static_cast<size_t>(kOperandBytes) + 7168 /*control block*/;
  static_assert(kStages >= 2, "pipeline needs at least two stages");
  static_assert(!kW8A16 || kLandingSlots >= 2, "W8A16 needs at least two landing slots");
  static_assert(!kW8A16 || kRowTile <= kBlockM, "token-major W8A16 holds an item's rows in the 128 lanes of one accumulator");
  static_assert(kAccColumns <= 512, "accumulator does not fit tensor memory");
};

// Per-column (= per token row) values of the current work unit, staged once by the epilogue warps so that the
// element loop reads shared memory instead of issuing a dependent global load per element.
struct ColumnMeta {
  float scale[256];      // activation scale of the row (int8)
  uint64_t rowptr[256];  // down / dense: byte address of the output row (may be peer memory)
};

struct SmemControl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t landed[8];        // W8A16: the int8 weight tile of a landing slot has arrived
  uint64_t landing_free[8];  // W8A16: every converter warp has read the slot
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  int last_part;           // dense split-K: this CTA holds the last part of its unit and finishes it
  uint32_t exp_table[64];  // copy of kExp2Table: divergent lookups are served by 32 banks
  ColumnMeta meta[2];
};

static_assert(sizeof(SmemControl) <= 7168, "control block exceeds its shared-memory reservation");

// Four int8 values (one 32-bit word) -> four bf16 values, exactly.  byte ^ 0x80 is the value + 128 as an unsigned
// byte; placed in the low mantissa bits of 2^23 it makes the float 2^23 + 128 + value, and subtracting 2^23 + 128
// leaves the value itself, whose upper 16 bits are its bf16 form (|value| <= 128 has at most 8 significant bits).
// (Both MMA operands stay bf16: an instruction descriptor that mixed an fp16 B operand with the bf16 A operand,
// which would halve this arithmetic, ended in a launch error on this driver and is not used.)
__device__ __forceinline__ void widen_int8x4(uint32_t word, uint32_t* low_pair, uint32_t* high_pair) {
  const uint32_t biased = word ^ 0x80808080u;
  const float magic = 8388736.0f;  // 2^23 + 128
  const float f0 = __fsub_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7540)), magic);
  const float f1 = __fsub_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7541)), magic);
  const float f2 = __fsub_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7542)), magic);
  const float f3 = __fsub_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7543)), magic);
  *low_pair = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
  *high_pair = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
}

// kPlanes (an instance of the int8 kernel; W8A16 in its fixed-point form): every activation row arrives as two int8
// rows, row 2p = the high plane and row 2p + 1 = the low plane of the row's 16-bit fixed-point values
// X = 256 * high + low, so a work item of r routes has 2r token rows and its accumulator columns come in pairs:
// the exact integer dot product of route p with a channel is 256 * column(2p) + column(2p + 1).  Work items are
// given in routes; loads, the MMA's N and the epilogue count plane rows.
template <bool kInt8, bool kGateUp, int kRowTile, bool kDense, bool kW8A16 = false, bool kPlanes = false>
__global__ void __launch_bounds__(kW8A16 ? kThreadsW8A16 : kThreads, 1)
umma_grouped_gemm_kernel(const __grid_constant__ CUtensorMap weight_map, const __grid_constant__ CUtensorMap token_map,
                         GroupedGemmArgs args) {
  static_assert(!kW8A16 || (!kInt8 && !kDense), "W8A16 is an instance of the bf16 grouped kernel");
  static_assert(!kPlanes || (kInt8 && !kDense && !kW8A16), "the two-plane form is an instance of the int8 grouped kernel");
  constexpr int kRowsPerRoute = kPlanes ? 2 : 1;
  using Cfg = TileConfig<kGateUp, kRowTile, kW8A16>;
  constexpr int kElemBytes = kInt8 ? 1 : 2;
  constexpr int kBlockKElems = kBlockKBytes / kElemBytes;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  SmemControl* ctl = reinterpret_cast<SmemControl*>(smem + static_cast<size_t>(Cfg::kOperandBytes));

  // Warp index, item count and (below) the tensor-memory base pass through a shuffle: the same values, but known to the
  // compiler as warp-uniform, which the warps that feed TMA and the tensor pipe need (ptx::elect_one).
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  int* status = args.status_rw;

  const int items = __shfl_sync(0xffffffffu, min(args.status[args.item_count_word], args.max_items), 0);
  const int n_blocks = (args.n_out + kBlockM - 1) / kBlockM;
  const int n_total = kGateUp ? 2 * args.n_out : args.n_out;
  const int64_t units = static_cast<int64_t>(items) * n_blocks;
  const int k_blocks = (args.k + kBlockKElems - 1) / kBlockKElems;
  // Dense split-K: `parts` work units per (row tile, channel block), part p over K blocks [p k_blocks / parts,
  // (p + 1) k_blocks / parts).  Everything else runs with parts == 1.
  const int parts = kDense ? (args.dense_splits > 1 ? args.dense_splits : 1) : 1;
  const int64_t part_units = units * parts;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      // W8A16: an operand stage is full when every converter warp has written its share of the bf16 weight tile.
      ptx::mbar_init(&ctl->full[s], kW8A16 ? kConvertWarps : 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int s = 0; s < 8; ++s) {
      ptx::mbar_init(&ctl->landed[s], 1);
      ptx::mbar_init(&ctl->landing_free[s], kConvertWarps + 1);  // the converter warps read the int8 tile, the MMAs the token tile
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&ctl->acc_full[b], 1);
      ptx::mbar_init(&ctl->acc_empty[b], 4);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
  }
  if (threadIdx.x >= 64 && threadIdx.x < 128) ctl->exp_table[threadIdx.x - 64] = kExp2Table[threadIdx.x - 64];
  if (warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, Cfg::kTmemColumns);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, ctl->tmem_base, 0);
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // The whole warp walks the loops; one elected lane issues the loads.
    {
      const bool issuer = ptx::elect_one();
      if (issuer) {
        ptx::prefetch_tensormap(&weight_map);
        ptx::prefetch_tensormap(&token_map);
      }
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      if constexpr (kW8A16) {
        // Landing producer: the token tile and the int8 weight tiles of every K block into the landing ring, as far
        // ahead as the ring allows.
        int slot = 0;
        uint32_t slot_phase = 0;
        int landed_issued = 0;
        for (int64_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
          int item, block;
          decode_unit(args.items, unit, n_blocks, &item, &block);
          item = __shfl_sync(0xffffffffu, item, 0);  // read from the item list: the same in every lane
          block = __shfl_sync(0xffffffffu, block, 0);
          const int weight_row = __shfl_sync(0xffffffffu, args.items[4 * item + 0], 0) * n_total + block * kBlockM;
          const int row0 = __shfl_sync(0xffffffffu, args.items[4 * item + 1], 0);
          for (int kb = 0; kb < k_blocks; ++kb) {
            ptx::mbar_wait(&ctl->landing_free[slot], slot_phase ^ 1u, abort_flag, status, 6);
            if (issuer) {
              uint8_t* landing = smem + Cfg::kLandingOffset + static_cast<size_t>(slot) * Cfg::kLandingBytes;
              const int x = kb * kBlockKElems;
              ptx::mbar_arrive_expect_tx(&ctl->landed[slot], Cfg::kTokenBytes + Cfg::kInt8TileBytes);
              ptx::tma_load_2d(landing, &token_map, &ctl->landed[slot], x, row0);
              ptx::tma_load_2d(landing + Cfg::kTokenRegionBytes, &weight_map, &ctl->landed[slot], x, weight_row);
              if (kGateUp) {
                ptx::tma_load_2d(landing + Cfg::kTokenRegionBytes + kBlockM * kLandingRowBytes, &weight_map, &ctl->landed[slot], x,
                                 weight_row + args.n_out);
              }
            }
            ++landed_issued;
            if (++slot == Cfg::kLandingSlots) {
              slot = 0;
              slot_phase ^= 1u;
            }
          }
        }
        // Drain (matters only after an abort): the loads issued last must have landed before the CTA exits.
        const int outstanding = landed_issued < Cfg::kLandingSlots ? landed_issued : Cfg::kLandingSlots;
        for (int back = 0; back < outstanding; ++back) {
          int sl = slot - 1 - back;
          uint32_t p = slot_phase;
          if (sl < 0) {
            sl += Cfg::kLandingSlots;
            p ^= 1u;
          }
          const unsigned long long start = ptx::global_timer_ns();
          while (!ptx::mbar_try_wait(&ctl->landed[sl], p)) {
            if (ptx::global_timer_ns() - start > ptx::kWaitLimitNs) break;
          }
        }
      }
      for (int64_t part_unit = blockIdx.x; !kW8A16 && part_unit < part_units; part_unit += gridDim.x) {
        const int64_t unit = part_unit / parts;
        const int part = static_cast<int>(part_unit - unit * parts);
        const int kb_begin = part * k_blocks / parts, kb_end = (part + 1) * k_blocks / parts;
        int item, block;
        decode_unit(args.items, unit, n_blocks, &item, &block);
        item = __shfl_sync(0xffffffffu, item, 0);  // read from the item list: the same in every lane
        block = __shfl_sync(0xffffffffu, block, 0);
        const int n0 = block * kBlockM;
        const int expert = __shfl_sync(0xffffffffu, args.items[4 * item + 0], 0);
        const int row0 = __shfl_sync(0xffffffffu, args.items[4 * item + 1], 0) * kRowsPerRoute;
        const int weight_row = expert * n_total + n0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ptx::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag, status, 1);
          uint8_t* stage_base = smem + static_cast<size_t>(stage) * Cfg::kStageBytes;
          if (!issuer) {
            // the other lanes only keep step
          } else if (FMOE_DIAG_BIT(args, 2)) {
            ptx::mbar_arrive(&ctl->full[stage]);
          } else {
            ptx::mbar_arrive_expect_tx(&ctl->full[stage], Cfg::kStageBytes);
            const int x = kb * kBlockKElems;
            ptx::tma_load_2d(stage_base, &weight_map, &ctl->full[stage], x, weight_row);
            if (kGateUp) ptx::tma_load_2d(stage_base + kBlockM * kBlockKBytes, &weight_map, &ctl->full[stage], x, weight_row + args.n_out);
            ptx::tma_load_2d(stage_base + Cfg::kWeightBytes, &token_map, &ctl->full[stage], x, row0);
          }
          ++issued;
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // Drain: every load this thread issued must have landed before the CTA may exit.  In a healthy
      // run the MMA warp has already consumed them; this only matters after an abort.
      const int pending = issued < Cfg::kStages ? issued : Cfg::kStages;
      for (int back = 0; back < pending; ++back) {
        int s = stage - 1 - back;
        uint32_t p = phase;
        if (s < 0) {
          s += Cfg::kStages;
          p ^= 1u;
        }
        const unsigned long long start = ptx::global_timer_ns();
        while (!ptx::mbar_try_wait(&ctl->full[s], p)) {
          if (ptx::global_timer_ns() - start > ptx::kWaitLimitNs) break;
        }
      }
    }
  } else if (kW8A16 && warp >= kConvertWarp0) {
    // ---------------- W8A16: widen the landed int8 weight tiles into the MMA's bf16 operand tiles ----------------
    // Per K block: wait until the operand stage is free (the MMAs that read it have completed) and the int8 tile has
    // landed; widen.
    // A row's 16-byte bf16 chunks go to the 128-byte-swizzled position the MMA descriptor expects (chunk index
    // XOR row mod 8).
    const int converter = static_cast<int>(threadIdx.x) - kConvertWarp0 * 32;
    constexpr int kUnits = Cfg::kWeightTiles * kBlockM * 4;  // 16-byte units of the int8 tile
    int stage = 0, slot = 0;
    uint32_t phase = 0, slot_phase = 0;
    for (int64_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        ptx::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag, status, 1);
        uint8_t* stage_base = smem + static_cast<size_t>(stage) * Cfg::kStageBytes;
        ptx::mbar_wait(&ctl->landed[slot], slot_phase, abort_flag, status, 5);
        const uint8_t* landing = smem + Cfg::kLandingOffset + static_cast<size_t>(slot) * Cfg::kLandingBytes + Cfg::kTokenRegionBytes;
        if (!FMOE_DIAG_BIT(args, 8)) {
          // Consecutive threads take consecutive 16-byte units (16 weights) of the landing slot: conflict-free
          // loads; the two 16-byte bf16 chunks of a unit go to swizzled positions that are conflict-free as well.
          uint4 packed[(kUnits + kConvertWarps * 32 - 1) / (kConvertWarps * 32)];
#pragma unroll
          for (int i = 0; i < static_cast<int>(sizeof(packed) / sizeof(packed[0])); ++i) {
            const int unit16 = converter + i * kConvertWarps * 32;
            if (unit16 < kUnits) packed[i] = reinterpret_cast<const uint4*>(landing)[unit16];
          }
#pragma unroll
          for (int i = 0; i < static_cast<int>(sizeof(packed) / sizeof(packed[0])); ++i) {
            const int unit16 = converter + i * kConvertWarps * 32;
            if (unit16 < kUnits) {
              const int row = unit16 >> 2;  // 0..127 gate (or the only) tile, 128..255 up tile: the tiles are contiguous
              const int chunk = (unit16 & 3) * 2;
              uint4 first, second;
              widen_int8x4(packed[i].x, &first.x, &first.y);
              widen_int8x4(packed[i].y, &first.z, &first.w);
              widen_int8x4(packed[i].z, &second.x, &second.y);
              widen_int8x4(packed[i].w, &second.z, &second.w);
              uint8_t* out_row = stage_base + row * kBlockKBytes;
              *reinterpret_cast<uint4*>(out_row + ((chunk ^ (row & 7)) << 4)) = first;
              *reinterpret_cast<uint4*>(out_row + (((chunk + 1) ^ (row & 7)) << 4)) = second;
            }
          }
        }
        // Generic-proxy writes must be visible to the tensor core's (async proxy) reads before the arrival.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(&ctl->full[stage]);
          ptx::mbar_arrive(&ctl->landing_free[slot]);
        }
        if (++stage == Cfg::kStages) {
          stage = 0;
          phase ^= 1u;
        }
        if (++slot == Cfg::kLandingSlots) {
          slot = 0;
          slot_phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the loop (waits included); one elected lane issues the MMAs and commits.
    {
      const bool issuer = ptx::elect_one();
      int stage = 0;
      uint32_t phase = 0;
      int slot = 0;  // W8A16: landing slot of the K block (its token tile is the MMA's B operand)
      int local = 0;
      for (int64_t part_unit = blockIdx.x; part_unit < part_units; part_unit += gridDim.x, ++local) {
        const int64_t unit = part_unit / parts;
        const int part = static_cast<int>(part_unit - unit * parts);
        const int kb_begin = part * k_blocks / parts, kb_end = (part + 1) * k_blocks / parts;
        const int buffer = local % Cfg::kAccBuffers;
        const uint32_t use = static_cast<uint32_t>(local / Cfg::kAccBuffers);
        // The MMA's N follows the rows this unit really has (multiple of 16): a tail item of a few rows costs a
        // few columns of tensor-core time, not a full tile.  Unused accumulator columns are never read.
        int item, block;
        decode_unit(args.items, unit, n_blocks, &item, &block);
        item = __shfl_sync(0xffffffffu, item, 0);  // read from the item list: the same in every lane
        block = __shfl_sync(0xffffffffu, block, 0);
        const int item_rows = __shfl_sync(0xffffffffu, args.items[4 * item + 2], 0) * kRowsPerRoute;
        const int mma_n = min(kRowTile, (item_rows + 15) & ~15);
        // Weight-major: M = 128 channels, N = the item's rows.  Token-major (W8A16): M = 128 token lanes, N = the
        // unit's channels (gate and up tiles are one 256-row B operand).
        const uint32_t idesc = kW8A16 ? ptx::make_instr_desc(false, kBlockM, Cfg::kWeightTiles * kBlockM) : ptx::make_instr_desc(kInt8, kBlockM, mma_n);
        ptx::mbar_wait(&ctl->acc_empty[buffer], (use & 1u) ^ 1u, abort_flag, status, 2);
        ptx::tcgen05_fence_after();
        const uint32_t acc = tmem_base + static_cast<uint32_t>(buffer * Cfg::kAccColumns);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          ptx::mbar_wait(&ctl->full[stage], phase, abort_flag, status, 3);
          ptx::tcgen05_fence_after();
          const uint32_t stage_addr = ptx::smem_u32(smem + static_cast<size_t>(stage) * Cfg::kStageBytes);
          // Token tile: behind the weight tile(s) of the stage, or (W8A16) at the head of the K block's landing slot.
          const uint32_t token_addr = kW8A16 ? ptx::smem_u32(smem + Cfg::kLandingOffset + static_cast<size_t>(slot) * Cfg::kLandingBytes)
                                             : stage_addr + Cfg::kWeightBytes;
#pragma unroll
          for (int ks = 0; ks < kBlockKBytes / kUmmaKBytes; ++ks) {
            if (FMOE_DIAG_BIT(args, 4) || !issuer) break;
            const uint64_t desc_gate = ptx::make_smem_desc_sw128(stage_addr + ks * kUmmaKBytes);
            const uint64_t desc_tok = ptx::make_smem_desc_sw128(token_addr + ks * kUmmaKBytes);
            const uint32_t accumulate = (kb > kb_begin || ks > 0) ? 1u : 0u;
            if constexpr (kW8A16) {
              ptx::umma_ss<false>(acc, desc_tok, desc_gate, idesc, accumulate);  // A = tokens, B = gate (+ up) channels
              continue;
            }
            ptx::umma_ss<kInt8>(acc, desc_gate, desc_tok, idesc, accumulate);
            if (kGateUp) {
              const uint64_t desc_up = ptx::make_smem_desc_sw128(stage_addr + kBlockM * kBlockKBytes + ks * kUmmaKBytes);
              ptx::umma_ss<kInt8>(acc + kRowTile, desc_up, desc_tok, idesc, accumulate);
            }
          }
          if (issuer) ptx::tcgen05_commit(&ctl->empty[stage]);  // frees the stage once these MMAs have read it
          if constexpr (kW8A16) {
            if (issuer) ptx::tcgen05_commit(&ctl->landing_free[slot]);  // ... and, with the converter warps' arrivals, the landing slot
            if (++slot == Cfg::kLandingSlots) slot = 0;
          }
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (issuer) ptx::tcgen05_commit(&ctl->acc_full[buffer]);  // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;  // the TMEM lanes a warp may read are fixed by warp id % 4
    const int channel_in_block = quarter * 32 + lane;
    const int epilogue_thread = static_cast<int>(threadIdx.x) - kEpilogueWarp0 * 32;
    const int n_out = args.n_out;
    const int numerics = args.numerics;
    const float limit = args.swiglu_limit;
    const int activation = args.activation;
    uint32_t* const dump = kPlanes ? nullptr : static_cast<uint32_t*>(args.dump_acc);  // the dump holds one row per route
    int local = 0;
    for (int64_t part_unit = blockIdx.x; part_unit < part_units; part_unit += gridDim.x, ++local) {
      const int64_t unit = part_unit / parts;
      const int buffer = local % Cfg::kAccBuffers;
      const uint32_t use = static_cast<uint32_t>(local / Cfg::kAccBuffers);
      int item, block;
      decode_unit(args.items, unit, n_blocks, &item, &block);
      item = __shfl_sync(0xffffffffu, item, 0);  // read from the item list: the same in every lane
      block = __shfl_sync(0xffffffffu, block, 0);
      const int n = block * kBlockM + channel_in_block;
      const int expert = args.items[4 * item + 0];
      const int row0 = args.items[4 * item + 1] * kRowsPerRoute;  // token rows (two per route in the two-plane form)
      const int rows = args.items[4 * item + 2] * kRowsPerRoute;
      const bool channel_ok = n < n_out;
      ColumnMeta* meta = &ctl->meta[local & 1];
      if constexpr (kW8A16) {
        // Token-major: this thread owns token row `channel_in_block` of the item (TMEM lane = token), the columns are
        // the unit's channels.  The per-channel scales of the unit go to shared memory first: scale[c] for the gate
        // (or only) tile's channel n0 + c, scale[128 + c] for the up tile's.
        const int n0 = block * kBlockM;
        {
          const float* s = args.w_scale + static_cast<int64_t>(expert) * n_total;
          meta->scale[epilogue_thread] = n0 + epilogue_thread < n_out ? s[n0 + epilogue_thread] : 0.0f;
          if (kGateUp) meta->scale[kBlockM + epilogue_thread] = n0 + epilogue_thread < n_out ? s[n_out + n0 + epilogue_thread] : 0.0f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        ptx::mbar_wait(&ctl->acc_full[buffer], use & 1u, abort_flag, status, 4);
        ptx::tcgen05_fence_after();
        const uint32_t acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buffer * Cfg::kAccColumns);
        const int token = channel_in_block;  // 0..127
        const bool row_ok = token < rows;
        const bool warp_has_rows = quarter * 32 < rows;  // warp-uniform: the tcgen05.ld below needs the whole warp
        const int channels = min(kBlockM, n_out - n0);   // a multiple of 16
        uint8_t* out_row = nullptr;
        if (row_ok) {
          if constexpr (kGateUp) {
            out_row = reinterpret_cast<uint8_t*>(args.y + static_cast<int64_t>(row0 + token) * n_out + n0);
          } else {
            const uint64_t base = args.row_out_ptrs != nullptr
                                      ? args.row_out_ptrs[row0 + token]
                                      : reinterpret_cast<uint64_t>(args.route_out) +
                                            static_cast<uint64_t>(args.sorted_routes[row0 + token]) * n_out * (args.route_out_bf16 ? 2 : 4);
            out_row = reinterpret_cast<uint8_t*>(base) + static_cast<size_t>(n0) * (args.route_out_bf16 ? 2 : 4);
          }
        }
        for (int c0 = 0; warp_has_rows && c0 < channels; c0 += 8) {
          uint32_t gate_bits[8];
          uint32_t up_bits[8];
          ptx::tmem_ld_x8(acc + c0, gate_bits);
          if (kGateUp) ptx::tmem_ld_x8(acc + kBlockM + c0, up_bits);
          ptx::tmem_ld_wait();
          if (!row_ok) continue;
          if constexpr (kGateUp) {
            uint32_t packed[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              uint16_t pair[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const float gate = __fmul_rn(__uint_as_float(gate_bits[j + h]), meta->scale[c0 + j + h]);
                const float up = __fmul_rn(__uint_as_float(up_bits[j + h]), meta->scale[kBlockM + c0 + j + h]);
                pair[h] = activation == FMOE_ACT_SILU ? swiglu_to_bf16_with(gate, up, limit, ctl->exp_table)
                                                      : other_activation_to_bf16(activation, gate, up);
              }
              packed[j >> 1] = static_cast<uint32_t>(pair[0]) | (static_cast<uint32_t>(pair[1]) << 16);
            }
            *reinterpret_cast<uint4*>(out_row + c0 * 2) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          } else {
            float values[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) values[j] = __fmul_rn(__uint_as_float(gate_bits[j]), meta->scale[c0 + j]);
            if (args.route_out_bf16) {
              uint32_t packed[4];
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                packed[j >> 1] = static_cast<uint32_t>(f32_to_bf16_bits(values[j])) | (static_cast<uint32_t>(f32_to_bf16_bits(values[j + 1])) << 16);
              }
              *reinterpret_cast<uint4*>(out_row + c0 * 2) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            } else {
              *reinterpret_cast<float4*>(out_row + c0 * 4) = make_float4(values[0], values[1], values[2], values[3]);
              *reinterpret_cast<float4*>(out_row + c0 * 4 + 16) = make_float4(values[4], values[5], values[6], values[7]);
            }
          }
        }
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctl->acc_empty[buffer]);
        continue;
      }
      for (int c = epilogue_thread; c < rows; c += 128) {
        const int route_row = (row0 + c) / kRowsPerRoute;  // sorted position of the column's route
        if (kInt8) meta->scale[c] = args.a_scale[route_row];
        if constexpr (kDense) {
          meta->rowptr[c] = reinterpret_cast<uint64_t>(args.dense_out) + static_cast<uint64_t>(row0 + c) * n_out * (args.dense_out_bf16 ? 2 : 4);
        } else if constexpr (!kGateUp) {
          meta->rowptr[c] = args.row_out_ptrs != nullptr
                                ? args.row_out_ptrs[route_row]
                                : reinterpret_cast<uint64_t>(args.route_out) +
                                      static_cast<uint64_t>(args.sorted_routes[route_row]) * n_out * (args.route_out_bf16 ? 2 : 4);
        }
      }
      float scale_gate = 1.0f, scale_up = 1.0f;
      if ((kInt8 || kW8A16) && channel_ok) {
        const float* s = args.w_scale + static_cast<int64_t>(expert) * n_total;
        scale_gate = s[n];
        if (kGateUp) scale_up = s[n + n_out];
      }
      float bias = 0.0f;
      if (kDense && channel_ok && args.bias != nullptr) bias = args.bias[n];
      float bias_gate = 0.0f, bias_up = 0.0f;  // per-expert bias of the BF16 path (gate_up: gate / up; down: bias_gate)
      if (!kInt8 && !kDense && channel_ok && args.expert_bias != nullptr) {
        const float* b = args.expert_bias + static_cast<int64_t>(expert) * n_total;
        bias_gate = b[n];
        if (kGateUp) bias_up = b[n + n_out];
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // metadata visible to the four epilogue warps
      ptx::mbar_wait(&ctl->acc_full[buffer], use & 1u, abort_flag, status, 4);
      ptx::tcgen05_fence_after();
      const uint32_t acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buffer * Cfg::kAccColumns);
      if constexpr (kDense) {
        if (parts > 1) {
          // This part's int32 sums go into the shared table; the part that finds the other parts' counts complete reads
          // the totals back and finishes the unit (integer addition: the order of the parts changes nothing).
          for (int c0 = 0; c0 < rows; c0 += 8) {
            uint32_t bits[8];
            ptx::tmem_ld_x8(acc + c0, bits);
            ptx::tmem_ld_wait();
            if (channel_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (c0 + j < rows) atomicAdd(args.dense_partial + static_cast<int64_t>(row0 + c0 + j) * n_out + n, static_cast<int>(bits[j]));
              }
            }
          }
          ptx::tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&ctl->acc_empty[buffer]);
          __threadfence();  // this thread's additions are visible before the count below
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (epilogue_thread == 0) ctl->last_part = atomicAdd(args.dense_counters + unit, 1) == parts - 1 ? 1 : 0;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (ctl->last_part) {
            __threadfence();  // the other parts' additions, published before their counts, are visible after ours
            if (channel_ok) {
              // Sixteen rows at a time: the loads of a batch are in flight together.
              for (int c0 = 0; c0 < rows; c0 += 16) {
                int totals[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  totals[j] = c0 + j < rows ? __ldcg(args.dense_partial + static_cast<int64_t>(row0 + c0 + j) * n_out + n) : 0;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  if (c0 + j >= rows) break;
                  const float value = __fadd_rn(dequantize(totals[j], meta->scale[c0 + j], scale_gate, numerics), bias);
                  const uint64_t rowptr = meta->rowptr[c0 + j];
                  if (args.dense_out_bf16) {
                    reinterpret_cast<uint16_t*>(rowptr)[n] = f32_to_bf16_bits(value);
                  } else {
                    reinterpret_cast<float*>(rowptr)[n] = value;
                  }
                }
              }
            }
          }
          continue;
        }
      }
      for (int c0 = 0; c0 < (FMOE_DIAG_BIT(args, 1) ? 0 : rows); c0 += 8) {
        uint32_t gate_bits[8];
        uint32_t up_bits[8];
        ptx::tmem_ld_x8(acc + c0, gate_bits);
        if (kGateUp) ptx::tmem_ld_x8(acc + kRowTile + c0, up_bits);
        ptx::tmem_ld_wait();
        if (channel_ok) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if constexpr (kPlanes) {
              // Columns (j, j + 1) = (high, low) plane of one route; rows is even, so the pair is complete.
              if ((j & 1) == 0 && c0 + j < rows) {
                const float a = meta->scale[c0 + j];
                if constexpr (kGateUp) {
                  const float gate = dequantize_planes(static_cast<int>(gate_bits[j]), static_cast<int>(gate_bits[j + 1]), a, scale_gate);
                  const float up = dequantize_planes(static_cast<int>(up_bits[j]), static_cast<int>(up_bits[j + 1]), a, scale_up);
                  args.y[static_cast<int64_t>((row0 + c0 + j) >> 1) * n_out + n] =
                      activation == FMOE_ACT_SILU ? swiglu_to_bf16_with(gate, up, limit, ctl->exp_table)
                                                  : other_activation_to_bf16(activation, gate, up);
                } else {
                  const float value = dequantize_planes(static_cast<int>(gate_bits[j]), static_cast<int>(gate_bits[j + 1]), a, scale_gate);
                  const uint64_t rowptr = meta->rowptr[c0 + j];
                  if (args.route_out_bf16) {
                    reinterpret_cast<uint16_t*>(rowptr)[n] = f32_to_bf16_bits(value);
                  } else {
                    reinterpret_cast<float*>(rowptr)[n] = value;
                  }
                }
              }
              continue;
            }
            if (c0 + j < rows) {
              if (dump != nullptr) {
                uint32_t* out = dump + static_cast<int64_t>(row0 + c0 + j) * n_total;
                out[n] = gate_bits[j];
                if (kGateUp) out[n + n_out] = up_bits[j];
              }
              if constexpr (kGateUp) {
                float gate, up;
                if constexpr (kInt8) {
                  const float a = meta->scale[c0 + j];
                  gate = dequantize(static_cast<int>(gate_bits[j]), a, scale_gate, numerics);
                  up = dequantize(static_cast<int>(up_bits[j]), a, scale_up, numerics);
                } else if constexpr (kW8A16) {
                  gate = __fmul_rn(__uint_as_float(gate_bits[j]), scale_gate);
                  up = __fmul_rn(__uint_as_float(up_bits[j]), scale_up);
                } else {
                  gate = __fadd_rn(__uint_as_float(gate_bits[j]), bias_gate);
                  up = __fadd_rn(__uint_as_float(up_bits[j]), bias_up);
                }
                args.y[static_cast<int64_t>(row0 + c0 + j) * n_out + n] =
                    (kInt8 || activation == FMOE_ACT_SILU) ? swiglu_to_bf16_with(gate, up, limit, ctl->exp_table)
                                                           : other_activation_to_bf16(activation, gate, up);
              } else {
                float value;
                if constexpr (kInt8) {
                  value = dequantize(static_cast<int>(gate_bits[j]), meta->scale[c0 + j], scale_gate, numerics);
                } else if constexpr (kW8A16) {
                  value = __fmul_rn(__uint_as_float(gate_bits[j]), scale_gate);
                } else {
                  value = __fadd_rn(__uint_as_float(gate_bits[j]), bias_gate);
                }
                const uint64_t rowptr = meta->rowptr[c0 + j];
                if constexpr (kDense) {
                  value = __fadd_rn(value, bias);
                  if (args.dense_out_bf16) {
                    reinterpret_cast<uint16_t*>(rowptr)[n] = f32_to_bf16_bits(value);
                  } else {
                    reinterpret_cast<float*>(rowptr)[n] = value;
                  }
                } else if (args.route_out_bf16) {
                  reinterpret_cast<uint16_t*>(rowptr)[n] = f32_to_bf16_bits(value);
                } else {
                  reinterpret_cast<float*>(rowptr)[n] = value;
                }
              }
            }
          }
        }
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&ctl->acc_empty[buffer]);
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemColumns);
  }
}

// ---- host side -------------------------------------------------------------------------------

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
  const CUresult result = encode(map, int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                 const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return result == CUDA_SUCCESS;
}

// W8A16 landing loads: int8 weight rows [rows, k] as plain (unswizzled) boxes of {64 bytes of K, 128 rows}.
bool make_landing_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {k};
  const cuuint32_t box[2] = {kLandingRowBytes, kBlockM};
  const cuuint32_t elem_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool kInt8, bool kGateUp, int kRowTile, bool kDense, bool kW8A16 = false, bool kPlanes = false>
cudaError_t launch_config(const GroupedGemmArgs& args, cudaStream_t stream) {
  using Cfg = TileConfig<kGateUp, kRowTile, kW8A16>;
  auto kernel = umma_grouped_gemm_kernel<kInt8, kGateUp, kRowTile, kDense, kW8A16, kPlanes>;
  static PerDeviceOnce configured;
  const int device = current_device_ordinal();
  if (configured.needed(device)) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmemBytes));
    if (err != cudaSuccess) return err;
    configured.mark(device);
  }
  const int n_total = kGateUp ? 2 * args.n_out : args.n_out;
  CUtensorMap weight_map, token_map;
  const bool weights_ok = kW8A16 ? make_landing_map(&weight_map, args.weights, static_cast<uint64_t>(args.experts) * n_total, args.k)
                                 : make_tensor_map(&weight_map, args.weights, kInt8, static_cast<uint64_t>(args.experts) * n_total, args.k, kBlockM);
  const uint64_t token_rows = static_cast<uint64_t>(args.total_rows) * (kPlanes ? 2 : 1);
  if (!weights_ok || !make_tensor_map(&token_map, args.a_rows, kInt8, token_rows, args.k, kRowTile)) {
    return cudaErrorInvalidValue;
  }
  const int n_blocks = (args.n_out + kBlockM - 1) / kBlockM;
  int64_t grid = static_cast<int64_t>(args.max_items) * n_blocks * (kDense && args.dense_splits > 1 ? args.dense_splits : 1);
  const int sms = sm_count_of_current_device();
  if (grid > sms) grid = sms;
  if (grid <= 0) return cudaSuccess;
  kernel<<<static_cast<unsigned>(grid), kW8A16 ? kThreadsW8A16 : kThreads, Cfg::kSmemBytes, stream>>>(weight_map, token_map, args);
  return cudaGetLastError();
}

template <bool kInt8, bool kGateUp, bool kDense, bool kW8A16 = false, bool kPlanes = false>
cudaError_t launch_tile(const GroupedGemmArgs& args, cudaStream_t stream) {
  switch (args.row_tile) {
    case 16: return launch_config<kInt8, kGateUp, 16, kDense, kW8A16, kPlanes>(args, stream);
    case 32: return launch_config<kInt8, kGateUp, 32, kDense, kW8A16, kPlanes>(args, stream);
    case 64: return launch_config<kInt8, kGateUp, 64, kDense, kW8A16, kPlanes>(args, stream);
    case 128: return launch_config<kInt8, kGateUp, 128, kDense, kW8A16, kPlanes>(args, stream);
    case 256:
      // Token-major W8A16 holds an item in the 128 lanes of one accumulator: no 256-row tile.
      if constexpr (kW8A16) {
        return cudaErrorInvalidValue;
      } else {
        return launch_config<kInt8, kGateUp, 256, kDense, kW8A16, kPlanes>(args, stream);
      }
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

bool umma_row_tile_supported(int row_tile) {
  return row_tile == 16 || row_tile == 32 || row_tile == 64 || row_tile == 128 || row_tile == 256 || row_tile == kPairRowTile;
}

cudaError_t launch_umma_grouped_gemm(const GroupedGemmArgs& caller_args, bool int8, bool gate_up, cudaStream_t stream) {
  GroupedGemmArgs args = caller_args;
#ifdef FMOE_DIAG
  const char* diag = getenv("FUSED_CPP_MOE_GEMM_DIAG");  // diagnostic library only: stage switches of GroupedGemmArgs::diag
  args.diag = diag ? atoi(diag) : 0;
#else
  args.diag = 0;
#endif
  if (args.max_items <= 0 || args.total_rows <= 0) return cudaSuccess;
  if (args.w8a16 == 2) {
    // int8 weights, activations as two int8 planes per route: the int8 one-SM kernel with paired accumulator columns;
    // row_tile counts plane rows (two per route).
    if (!int8 || args.dense_out != nullptr || args.w_scale == nullptr || args.a_scale == nullptr) return cudaErrorInvalidValue;
    if (args.row_tile == kPairRowTile) return launch_umma_pair_grouped_gemm(args, true, gate_up, stream);  // items of at most 128 routes
    return gate_up ? launch_tile<true, true, false, false, true>(args, stream) : launch_tile<true, false, false, false, true>(args, stream);
  }
  if (args.w8a16) {
    // int8 weights with bf16 activations: the one-SM kernel with its widening warps, for every row tile.
    if (int8 || args.dense_out != nullptr || args.w_scale == nullptr) return cudaErrorInvalidValue;
    if (args.row_tile > 128) return cudaErrorInvalidValue;  // the caller caps W8A16 work items at 128 rows
    return gate_up ? launch_tile<false, true, false, true>(args, stream) : launch_tile<false, false, false, true>(args, stream);
  }
  if (args.row_tile == kPairRowTile) {
    if (umma_pair_supported(gate_up, args.n_out, args.total_rows)) return launch_umma_pair_grouped_gemm(args, int8, gate_up, stream);
    args.row_tile = 256;  // same 256-row work items, one-SM kernel
  }
  if (args.dense_out != nullptr) {
    if (!int8 || gate_up) return cudaErrorInvalidValue;  // the dense epilogue exists for the int8 single-stage GEMM
    return launch_tile<true, false, true>(args, stream);
  }
  if (int8) return gate_up ? launch_tile<true, true, false>(args, stream) : launch_tile<true, false, false>(args, stream);
  return gate_up ? launch_tile<false, true, false>(args, stream) : launch_tile<false, false, false>(args, stream);
}

}  // namespace fmoe
