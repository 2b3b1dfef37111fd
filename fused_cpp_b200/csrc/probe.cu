// Tensor-core issue-rate probe: every SM issues back-to-back tcgen05.mma on whatever its shared memory
// holds and the host times the launch.  It gives the dense MMA peak of this GPU for a tile shape
// (kind::i8 has no published measured figure on this part), the denominator for "fraction of the tensor
// roofline" in the prefill regime.  No global memory is touched; results are discarded.
// mode bit 0 fills the operands with a non-zero pattern instead of zeros (zero operands toggle few wires and
// draw less power than real data, so they give the rate at full clock rather than a sustainable one);
// mode >> 8 = c > 0 commits to an mbarrier after every c MMAs, the cadence of a pipelined GEMM main loop;
// mode bit 1 lets a second thread (warp 1) issue the same chain into a second accumulator at the same time, and
// mode bit 2 makes the one issuing thread alternate between the two accumulators (two independent chains): they
// tell a limit of the issuing thread from one of the tensor pipe;
// mode bit 4 (with c = mode >> 8): rounds of c MMAs, one commit and a wait for it: the latency of one pipeline stage.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace fmoe {

namespace {

template <bool kInt8>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int n, int iterations, int mode, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t done;
  __shared__ uint64_t cadence;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  // Operands must be finite for the f16 kind; zero everything.
  for (int i = threadIdx.x; i < (16384 + 32768) / 16; i += blockDim.x) {
    // Non-zero fill: bytes in [0, 63], i.e. small int8 values or finite bf16 values below 1.
    const uint32_t h = (mode & 1) ? ((static_cast<uint32_t>(i) * 2654435761u) >> 7) & 0x3f3f3f3fu : 0u;
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(h, h ^ 0x15150a0au, h ^ 0x2a0a2a15u, h ^ 0x0f0f3030u);
  }
  if (threadIdx.x == 0) {
    ptx::mbar_init(&done, (mode & 2) ? 2 : 1);
    ptx::mbar_init(&cadence, 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base, 512);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const bool second_issuer = (mode & 2) != 0;
  const bool alternate = (mode & 4) != 0;
  // The issuing warp(s) walk the loop as a whole and one elected lane issues (ptx::elect_one): what the GEMM kernels do.
  if (warp == 0 || (second_issuer && warp == 1)) {
    const bool issuer = ptx::elect_one();
    const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t a = ptx::smem_u32(smem);
    const uint32_t b = a + 16384;
    const uint32_t idesc = ptx::make_instr_desc(kInt8, 128, n);
    const int commit_every = mode >> 8;
    const uint32_t accumulator = tmem + (warp == 1 ? 256u : 0u);
    const int mine = second_issuer ? iterations / 2 : iterations;  // the same number of MMAs per launch in every mode
    if (mode & 16) {
      // Round trips: c MMAs, one commit, wait for it; the time per round is the latency of a pipeline stage of c MMAs.
      const int rounds = iterations / commit_every;
      for (int r = 0; r < rounds; ++r) {
        for (int j = 0; j < commit_every; ++j) {
          const uint32_t k = static_cast<uint32_t>(j & 3) * 32;
          if (issuer) ptx::umma_ss<kInt8>(accumulator, ptx::make_smem_desc_sw128(a + k), ptx::make_smem_desc_sw128(b + k), idesc, j > 0 ? 1u : 0u);
        }
        if (issuer) ptx::tcgen05_commit(&cadence);
        if (!ptx::mbar_wait_spin(&cadence, static_cast<uint32_t>(r) & 1u, &abort_flag, status, 33)) break;
        ptx::tcgen05_fence_after();
      }
    } else
    for (int i = 0; i < mine; ++i) {
      const uint32_t k = static_cast<uint32_t>(i & 3) * 32;
      const uint32_t target = accumulator + ((alternate && (i & 1)) ? 256u : 0u);
      if (issuer) ptx::umma_ss<kInt8>(target, ptx::make_smem_desc_sw128(a + k), ptx::make_smem_desc_sw128(b + k), idesc, i > 1 ? 1u : 0u);
      if (issuer && commit_every > 0 && ((i + 1) & (commit_every - 1)) == 0) ptx::tcgen05_commit(&cadence);  // c: a power of two
    }
    if (issuer) ptx::tcgen05_commit(&done);
    ptx::mbar_wait(&done, 0, &abort_flag, status, 31);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

template <bool kInt8>
__device__ __forceinline__ void pair_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  if constexpr (kInt8) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d), "l"(desc_a),
                 "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
  } else {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d), "l"(desc_a),
                 "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
  }
}

__device__ __forceinline__ void pair_commit(uint32_t cluster_address) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_address) : "memory");
}

// The same chain issued by the leader of a two-CTA cluster as tcgen05.mma.cta_group::2 of 256 x n x 32 bytes (every
// CTA holds 128 A rows and n / 2 B rows in its shared memory).  mode >> 8 = c > 0: after every c MMAs the leader commits
// to one mbarrier in each of the two CTAs, the cadence of the two-SM grouped GEMM's main loop.  Mode bits 1 and 2 as in
// the one-SM probe.
template <bool kInt8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) mma_rate_pair_kernel(int n, int iterations, int mode, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t done;
  __shared__ uint64_t cadence;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  uint32_t cta;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta));
  for (int i = threadIdx.x; i < (16384 + 16384) / 16; i += blockDim.x) {
    const uint32_t h = (mode & 1) ? ((static_cast<uint32_t>(i) * 2654435761u) >> 7) & 0x3f3f3f3fu : 0u;
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(h, h ^ 0x15150a0au, h ^ 0x2a0a2a15u, h ^ 0x0f0f3030u);
  }
  const bool second_issuer = (mode & 2) != 0;  // as in the one-SM probe: thread 32 of the leader issues half of the chain
  const bool alternate = (mode & 4) != 0;      // the issuing thread alternates between two accumulators
  if (threadIdx.x == 0) {
    ptx::mbar_init(&done, second_issuer ? 2 : 1);
    ptx::mbar_init(&cadence, 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(&tmem_base)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  ptx::tcgen05_fence_after();
  if (cta == 0 && (warp == 0 || (second_issuer && warp == 1))) {
    const bool issuer = ptx::elect_one();
    const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t a = ptx::smem_u32(smem);
    const uint32_t b = a + 16384;
    const uint32_t idesc = ptx::make_instr_desc(kInt8, 256, n);
    const int commit_every = mode >> 8;
    const uint32_t accumulator = tmem + (warp == 1 ? 256u : 0u);
    const int mine = second_issuer ? iterations / 2 : iterations;
    uint32_t cadence0, cadence1, done0;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(cadence0) : "r"(ptx::smem_u32(&cadence)), "r"(0u));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(cadence1) : "r"(ptx::smem_u32(&cadence)), "r"(1u));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(done0) : "r"(ptx::smem_u32(&done)), "r"(0u));
    if (mode & 16) {
      const int rounds = iterations / commit_every;
      for (int r = 0; r < rounds; ++r) {
        for (int j = 0; j < commit_every; ++j) {
          const uint32_t k = static_cast<uint32_t>(j & 3) * 32;
          if (issuer) pair_mma<kInt8>(accumulator, ptx::make_smem_desc_sw128(a + k), ptx::make_smem_desc_sw128(b + k), idesc, j > 0 ? 1u : 0u);
        }
        if (issuer) pair_commit(cadence0);
        if (!ptx::mbar_wait_spin(&cadence, static_cast<uint32_t>(r) & 1u, &abort_flag, status, 34)) break;
        ptx::tcgen05_fence_after();
      }
    } else {
      for (int i = 0; i < mine; ++i) {
        const uint32_t k = static_cast<uint32_t>(i & 3) * 32;
        const uint32_t target = accumulator + ((alternate && (i & 1)) ? 256u : 0u);
        if (issuer) pair_mma<kInt8>(target, ptx::make_smem_desc_sw128(a + k), ptx::make_smem_desc_sw128(b + k), idesc, i > 1 ? 1u : 0u);
        if (issuer && commit_every > 0 && ((i + 1) & (commit_every - 1)) == 0) {  // c: a power of two
          pair_commit(cadence0);
          if (!(mode & 32)) pair_commit(cadence1);
        }
      }
    }
    if (issuer) pair_commit(done0);
    ptx::mbar_wait(&done, 0, &abort_flag, status, 32);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  // Neither CTA leaves (or frees tensor memory) while the other may still read its operands.
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (warp == 0) {
    ptx::tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace

cudaError_t launch_mma_rate_probe(bool int8, int n, int iterations, int mode, int blocks, int* status, cudaStream_t stream) {
  const size_t smem = 1024 + 16384 + 32768;
  auto kernel = int8 ? mma_rate_kernel<true> : mma_rate_kernel<false>;
  cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (error != cudaSuccess) return error;
  kernel<<<blocks, 128, smem, stream>>>(n, iterations, mode, status);
  return cudaGetLastError();
}

cudaError_t launch_mma_rate_pair_probe(bool int8, int n, int iterations, int mode, int blocks, int* status, cudaStream_t stream) {
  const size_t smem = 1024 + 16384 + 16384;
  auto kernel = int8 ? mma_rate_pair_kernel<true> : mma_rate_pair_kernel<false>;
  cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (error != cudaSuccess) return error;
  kernel<<<blocks & ~1, 128, smem, stream>>>(n, iterations, mode, status);
  return cudaGetLastError();
}

}  // namespace fmoe
