// Tensor-core issue-rate probe: every SM issues back-to-back tcgen05.mma on whatever its shared memory
// holds and the host times the launch.  It gives the dense MMA peak of this GPU for a tile shape
// (kind::i8 has no published measured figure on this part), the denominator for "fraction of the tensor
// roofline" in the prefill regime.  No global memory is touched; results are discarded.
// mode bit 0 fills the operands with a non-zero pattern instead of zeros (zero operands toggle few wires and
// draw less power than real data, so they give the rate at full clock rather than a sustainable one);
// mode >> 8 = c > 0 commits to an mbarrier after every c MMAs, the cadence of a pipelined GEMM main loop.
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
  const int warp = threadIdx.x >> 5;
  // Operands must be finite for the f16 kind; zero everything.
  for (int i = threadIdx.x; i < (16384 + 32768) / 16; i += blockDim.x) {
    // Non-zero fill: bytes in [0, 63], i.e. small int8 values or finite bf16 values below 1.
    const uint32_t h = (mode & 1) ? ((static_cast<uint32_t>(i) * 2654435761u) >> 7) & 0x3f3f3f3fu : 0u;
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(h, h ^ 0x15150a0au, h ^ 0x2a0a2a15u, h ^ 0x0f0f3030u);
  }
  if (threadIdx.x == 0) {
    ptx::mbar_init(&done, 1);
    ptx::mbar_init(&cadence, 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base, 256);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  if (threadIdx.x == 0) {
    const uint32_t a = ptx::smem_u32(smem);
    const uint32_t b = a + 16384;
    const uint32_t idesc = ptx::make_instr_desc(kInt8, 128, n);
    const int commit_every = mode >> 8;
    for (int i = 0; i < iterations; ++i) {
      const uint32_t k = static_cast<uint32_t>(i & 3) * 32;
      ptx::umma_ss<kInt8>(tmem_base, ptx::make_smem_desc_sw128(a + k), ptx::make_smem_desc_sw128(b + k), idesc, i > 0 ? 1u : 0u);
      if (commit_every > 0 && (i + 1) % commit_every == 0) ptx::tcgen05_commit(&cadence);
    }
    ptx::tcgen05_commit(&done);
    ptx::mbar_wait(&done, 0, &abort_flag, status, 31);
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, 256);
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

}  // namespace fmoe
