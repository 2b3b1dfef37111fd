// Entry points and constants of the diagnostic library only (libfused_moe_b200_diag.so, built with -DFMOE_DIAG).
// The product library exports none of this and has one grouped-GEMM implementation (tcgen05).
#pragma once

#include "../../include/fused_moe_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* fmoe_config.gemm_impl = 1: a CUDA-core (dp4a / FMA) grouped GEMM used as a stage-level cross-check of the
 * tensor-core kernels, in the spirit of the reference's fused_moe_test_* hooks (csrc/moe/module.cpp:41-115). */
#define FMOE_GEMM_SIMT 1

/* Dense tensor-core issue rate of the current GPU for one MMA shape: every SM issues `iterations` back-to-back
 * tcgen05.mma of 128 x n x 32 bytes (kind::i8 when int8 != 0, else kind::f16 with bf16 operands) on shared
 * memory that is zeroed (mode bit 0 clear) or filled with a non-zero pattern (bit 0 set); mode >> 8 = c > 0 adds
 * a tcgen05.commit after every c MMAs; mode bit 1: a second thread issues half of the MMAs
 * into a second accumulator; bit 2: the issuing thread alternates between two accumulators; bit 3: two-SM MMAs of
 * 256 x n x 32 bytes issued by the leader of every two-CTA cluster (commits go to one barrier in each CTA).  Returns tera-operations per second (2 per multiply-add), best of three
 * timed launches.  Allocates a few bytes and synchronises. */
FMOE_API int fmoe_probe_mma_rate(int32_t int8, int32_t n, int32_t iterations, int32_t mode, float* tera_ops_per_s);

#ifdef __cplusplus
}
#endif
