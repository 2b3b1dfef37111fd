// Thin wrappers over the sm_100a instructions the grouped GEMM uses: mbarrier, TMA tiled loads,
// tensor-memory allocation, tcgen05.mma / commit / ld and the matching fences.
//
// Every wait is bounded: after kWaitLimitNs of polling it records FMOE_ERR_DEVICE_WAIT in the status
// block, raises the CTA-wide abort flag and returns, and every later wait returns at once, so a
// broken pipeline ends in an error code instead of a hung SM.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace fmoe {
namespace ptx {

constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // one second

__device__ __forceinline__ uint32_t smem_u32(const void* pointer) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long value;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(value));
  return value;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// One lane of the (converged) warp: true in exactly one lane.  Code that feeds tcgen05.mma / TMA should keep the whole
// warp in the loop and predicate only the issuing instructions with this flag: addresses, descriptors and counters then
// stay warp-uniform, and the compiler can hold them in the uniform registers those instructions read.  Inside a
// `lane == 0` branch every operand has to be moved over from ordinary registers each time.
__device__ __forceinline__ bool elect_one() {
  uint32_t elected;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(elected));
  return elected != 0;
}

// Non-blocking test of a phase (mbarrier.try_wait may park the thread for a while before it answers).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  Returns true when the phase completed, false when the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int site) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = global_timer_ns();
  while (true) {
    for (int spin = 0; spin < 64; ++spin) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag) return false;
    if (global_timer_ns() - start > kWaitLimitNs) {
      *abort_flag = 1;
      if (atomicCAS(status + kStatusError, 0, FMOE_ERR_DEVICE_WAIT) == 0) {
        status[kStatusDetail] = static_cast<int>(blockIdx.x);
        status[kStatusWaitSite] = site;
      }
      return false;
    }
  }
}

// The same bounded wait, polling with test_wait: for the one or two threads of a CTA whose wake-up latency is on the
// critical path of the pipeline.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int site) {
  if (mbar_test_wait(bar, parity)) return true;
  const unsigned long long start = global_timer_ns();
  while (true) {
    for (int spin = 0; spin < 256; ++spin) {
      if (mbar_test_wait(bar, parity)) return true;
    }
    if (*abort_flag) return false;
    if (global_timer_ns() - start > kWaitLimitNs) {
      *abort_flag = 1;
      if (atomicCAS(status + kStatusError, 0, FMOE_ERR_DEVICE_WAIT) == 0) {
        status[kStatusDetail] = static_cast<int>(blockIdx.x);
        status[kStatusWaitSite] = site;
      }
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory ---------------------------------------------------------------------------

// Whole-warp calls.  `columns` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// The mbarrier gets one arrival once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor for a K-major tile stored as 128-byte rows with the 128-byte
// swizzle (what a TMA tiled load with CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024
// bytes apart (stride-byte-offset field), the leading-byte-offset field is unused for swizzled
// K-major layouts and set to 1, descriptor version 1, layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_address) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_address & 0x3ffffu) >> 4);  // start address, bits [0,14)
  desc |= static_cast<uint64_t>(1) << 16;                         // leading byte offset (ignored), bits [16,30)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;                 // stride byte offset, bits [32,46)
  desc |= static_cast<uint64_t>(1) << 46;                         // descriptor version, bits [46,48)
  desc |= static_cast<uint64_t>(2) << 61;                         // SWIZZLE_128B, bits [61,64)
  return desc;
}

// Instruction descriptor of a dense cta_group::1 MMA, both operands K-major.
//   bits [4,6) accumulator format (1 = f32, 2 = s32); [7,10) A format; [10,13) B format
//   (kind::f16: 1 = bf16; kind::i8: 1 = signed int8); [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_instr_desc(bool int8, int m, int n) {
  return (static_cast<uint32_t>(int8 ? 2 : 1) << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; `accumulate` = 0 overwrites D.
template <bool kInt8>
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  if constexpr (kInt8) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Eight consecutive 32-bit columns of this thread's TMEM lane (the warp covers 32 lanes).
__device__ __forceinline__ void tmem_ld_x8(uint32_t address, uint32_t* v) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(address)
               : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace ptx
}  // namespace fmoe
