// Shared device helpers for the routed-expert MoE kernels (sm_100a).
//
// Arithmetic follows the reference CPU implementation statement by statement; every rounding step
// is spelled with a round-to-nearest intrinsic so that the compiler can neither fuse nor reorder it:
//   row quantiser      csrc/moe/arm/i8mm_w8a8/kernels.cpp:211-228 (NATIVE), tests/test_moe_w8a8.py:40-43 (TORCHREF)
//   exp(-gate)         csrc/moe/arm/i8mm_w8a8/kernels.cpp:200-209
//   clamped SwiGLU     csrc/moe/arm/i8mm_w8a8/kernels.cpp:230-246
//   bf16 store         csrc/moe/arm/i8mm_w8a8/kernels.cpp:194-198
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fused_moe_b200.h"

namespace fmoe {

// Layout of the status block at the start of every workspace (int32 words).
enum StatusWord : int {
  kStatusError = 0,      // first error code raised by a kernel (0 = none)
  kStatusDetail = 1,     // detail of that error (e.g. the offending flat route id)
  kStatusItems = 2,      // number of (expert, row-tile) work items of this call
  kStatusActive = 3,     // number of experts with at least one route
  kStatusWaitSite = 4,   // which bounded wait gave up (0 = none)
  kStatusItemsB = 5,     // work items of the second list (down GEMM)
  kStatusItemsC = 6,     // split mode: gate_up work items of the experts with many rows (two-SM kernel)
  kStatusItemsD = 7,     // split mode: down work items of those experts
  kStatusWords = 16,
};

__device__ __forceinline__ void raise_error(int* status, int code, int detail) {
  if (atomicCAS(status + kStatusError, 0, code) == 0) status[kStatusDetail] = detail;
}

// Work unit -> (work item, channel block).  Items are sorted by (expert, row tile); units are ordered so that,
// inside one expert, the row tiles of a channel block are adjacent: CTAs that run side by side then read the
// same weight tile at the same time and the second read is served by L2 instead of HBM.  items[4*i+3] packs
// the first item of the item's expert (20 bits) and that expert's tile count.
__device__ __forceinline__ void decode_unit(const int* __restrict__ items, int64_t unit, int n_blocks, int* item, int* block) {
  const int guess = static_cast<int>(unit / n_blocks);
  const int packed = items[4 * guess + 3];
  const int first = packed & 0xfffff;
  const int tiles = packed >> 20;
  const int64_t local = unit - static_cast<int64_t>(first) * n_blocks;
  *block = static_cast<int>(local / tiles);
  *item = first + static_cast<int>(local % tiles);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t bits) { return __uint_as_float(static_cast<uint32_t>(bits) << 16); }

// Nearest-even bf16 by adding 0x7fff + lsb, like the reference's store_bf16.
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float value) {
  const uint32_t bits = __float_as_uint(value);
  const uint32_t lsb = (bits >> 16) & 1u;
  return static_cast<uint16_t>((bits + 0x7fffu + lsb) >> 16);
}

// fp32(2^(i/64)): the significand table of the FEXPA instruction.
__device__ __constant__ const uint32_t kExp2Table[64] = {
    0x3f800000u, 0x3f8164d2u, 0x3f82cd87u, 0x3f843a29u, 0x3f85aac3u, 0x3f871f62u, 0x3f88980fu, 0x3f8a14d5u,
    0x3f8b95c2u, 0x3f8d1adfu, 0x3f8ea43au, 0x3f9031dcu, 0x3f91c3d3u, 0x3f935a2bu, 0x3f94f4f0u, 0x3f96942du,
    0x3f9837f0u, 0x3f99e046u, 0x3f9b8d3au, 0x3f9d3edau, 0x3f9ef532u, 0x3fa0b051u, 0x3fa27043u, 0x3fa43516u,
    0x3fa5fed7u, 0x3fa7cd94u, 0x3fa9a15bu, 0x3fab7a3au, 0x3fad583fu, 0x3faf3b79u, 0x3fb123f6u, 0x3fb311c4u,
    0x3fb504f3u, 0x3fb6fd92u, 0x3fb8fbafu, 0x3fbaff5bu, 0x3fbd08a4u, 0x3fbf179au, 0x3fc12c4du, 0x3fc346cdu,
    0x3fc5672au, 0x3fc78d75u, 0x3fc9b9beu, 0x3fcbec15u, 0x3fce248cu, 0x3fd06334u, 0x3fd2a81eu, 0x3fd4f35bu,
    0x3fd744fdu, 0x3fd99d16u, 0x3fdbfbb8u, 0x3fde60f5u, 0x3fe0ccdfu, 0x3fe33f89u, 0x3fe5b907u, 0x3fe8396au,
    0x3feac0c7u, 0x3fed4f30u, 0x3fefe4bau, 0x3ff28177u, 0x3ff5257du, 0x3ff7d0dfu, 0x3ffa83b3u, 0x3ffd3e0cu,
};

// exp(-gate) with the reference's FEXPA evaluator: range reduction to multiples of 1/64 in the
// exponent, a table significand and a degree-2 correction.  `table` is kExp2Table or a copy of it in
// shared memory: lanes index it with different values, which the constant cache serialises (one
// address per pass) while shared memory serves 32 banks at once.
__device__ __forceinline__ float expneg_with(float gate, const uint32_t* table) {
  float x = -gate;
  x = fminf(x, 87.0f);
  x = fmaxf(x, -87.0f);
  const float encoded = __fmaf_rn(x, 1.4426950216293335f, 196735.0f);
  const float k = __fsub_rn(encoded, 196735.0f);
  float residual = __fmaf_rn(-k, 0.693145751953125f, x);
  residual = __fmaf_rn(-k, 1.428606765330187e-06f, residual);
  const uint32_t enc_bits = __float_as_uint(encoded);
  const uint32_t scale_bits = (((enc_bits >> 6) & 0xffu) << 23) | (table[enc_bits & 63u] & 0x007fffffu);
  const float scale = __uint_as_float(scale_bits);
  const float polynomial = __fmaf_rn(residual, 0.5000003576278687f, 1.000003695487976f);
  return __fmaf_rn(scale, __fmul_rn(polynomial, residual), scale);
}

__device__ __forceinline__ float expneg(float gate) { return expneg_with(gate, kExp2Table); }

// (gate*up)/(exp(-gate)+1) -> bf16, with the optional +-limit clamp (limit <= 0: none).
__device__ __forceinline__ uint16_t swiglu_to_bf16_with(float gate, float up, float limit, const uint32_t* table) {
  if (limit > 0.0f) {
    gate = fminf(gate, limit);
    up = fmaxf(fminf(up, limit), -limit);
  }
  const float value = __fdiv_rn(__fmul_rn(gate, up), __fadd_rn(expneg_with(gate, table), 1.0f));
  return f32_to_bf16_bits(value);
}

// The other gated activations of the reference's BF16 op (csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:1911-1936,
// arithmetic as in src/fused_cpp/moe/naive.py:28-54).  Rare paths: kept out of line so that the SiLU loops do not
// carry their registers.
//   gelu:      0.5 * gate * (1 + erf(gate / sqrt(2))) * up
//   swigluoai: gate = min(gate, 7), up = clamp(up, +-7), (up + 1) * gate * sigmoid(1.702 * gate)
#define FMOE_ACT_SILU 0
#define FMOE_ACT_GELU 2
#define FMOE_ACT_SWIGLUOAI 3
static __device__ __noinline__ uint16_t other_activation_to_bf16(int activation, float gate, float up) {
  float value;
  if (activation == FMOE_ACT_GELU) {
    value = 0.5f * gate * (1.0f + erff(gate * 0.70710678118654752440f)) * up;
  } else {
    gate = fminf(gate, 7.0f);
    up = fmaxf(fminf(up, 7.0f), -7.0f);
    const float glu = gate / (1.0f + expf(-1.702f * gate));
    value = (up + 1.0f) * glu;
  }
  return f32_to_bf16_bits(value);
}

__device__ __forceinline__ uint16_t swiglu_to_bf16(float gate, float up, float limit) {
  return swiglu_to_bf16_with(gate, up, limit, kExp2Table);
}

// int32 accumulator -> fp32 with the activation and per-channel weight scale.
__device__ __forceinline__ float dequantize(int32_t accumulator, float activation_scale, float channel_scale, int numerics) {
  const float value = static_cast<float>(accumulator);  // cvt.rn.f32.s32
  if (numerics == FMOE_NUMERICS_NATIVE) return __fmul_rn(value, __fmul_rn(activation_scale, channel_scale));
  return __fmul_rn(__fmul_rn(value, activation_scale), channel_scale);
}

// Two-plane (16-bit fixed point) activations.  A row's values are X = rint(x / scale), scale = amax / kPlaneFullScale
// (1 for an all-zero row), |X| <= 32512 = 127 * 256, carried as X = 256 * high + low with low in [-128, 127] and high
// in [-127, 127].  The exact integer dot product with an int8 weight row is 256 * acc(high) + acc(low) (below 2^37 in
// magnitude); it is rounded to fp32 once, then scaled by the row scale and the channel scale in that order.
constexpr float kPlaneFullScale = 32512.0f;

__device__ __forceinline__ float plane_row_scale(float amax) { return amax > 0.0f ? __fdiv_rn(amax, kPlaneFullScale) : 1.0f; }

__device__ __forceinline__ int plane_fixed_point(float value, float scale) {
  const float rounded = rintf(__fdiv_rn(value, scale));  // ties to even
  return static_cast<int>(fmaxf(fminf(rounded, kPlaneFullScale), -kPlaneFullScale));
}

__device__ __forceinline__ float dequantize_planes(int32_t high, int32_t low, float activation_scale, float channel_scale) {
  const long long exact = static_cast<long long>(high) * 256 + static_cast<long long>(low);
  return __fmul_rn(__fmul_rn(__ll2float_rn(exact), activation_scale), channel_scale);
}

__device__ __forceinline__ float row_scale_from_amax(float amax, int numerics) {
  if (numerics == FMOE_NUMERICS_NATIVE) return amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
  const float scale = __fdiv_rn(amax, 127.0f);
  return scale < 1.0e-30f ? 1.0e-30f : scale;
}

// One activation value -> int8.  `scale_or_inverse` is 1/scale for NATIVE and scale for TORCHREF.
__device__ __forceinline__ int quantize_value(float value, float scale_or_inverse, int numerics) {
  if (numerics == FMOE_NUMERICS_NATIVE) {
    float scaled = __fmul_rn(value, scale_or_inverse);
    scaled = fmaxf(fminf(scaled, 127.0f), -127.0f);
    return static_cast<int>(roundf(scaled));  // ties away from zero
  }
  float rounded = rintf(__fdiv_rn(value, scale_or_inverse));  // ties to even
  rounded = fmaxf(fminf(rounded, 127.0f), -127.0f);
  return static_cast<int>(rounded);
}

// TORCHREF quantisation of four values with the division replaced by a multiplication wherever that cannot change
// the result.  value * (1/scale) differs from the correctly rounded value / scale by at most a few units in the
// last place (below 4e-5 in absolute terms for |quotient| <= 128), so the two round to the same integer unless
// the product lies within 1e-4 of a half-integer; only then the exact division decides.  Bit-identical to
// quantize_value(TORCHREF).  The conversions are taken out of the common path as well.  The product is clamped
// first (rint and a clamp at the integers +-127 commute; the order of fminf / fmaxf is quantize_value's, so NaN ends
// at +127 there too); adding 1.5 * 2^23 rounds it to the nearest integer, ties to even, in the low mantissa bits, so
// the byte is read out of the sum's bit pattern and subtracting the constant again gives rint(product) for the
// boundary test: no FRND and no F2I, which issue at a quarter of the FADD rate.  A clamped product is an integer
// (distance 0) and the exact quotient then rounds to +-127 as well.  One test per four values; the exact division
// decides all four when any of them is near a boundary.
__device__ __forceinline__ uint32_t quantize4_torchref_fast(const float* values, float scale, float inverse) {
  constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
  uint32_t bits[4];
  float worst = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float product = fmaxf(fminf(__fmul_rn(values[i], inverse), 127.0f), -127.0f);
    const float shifted = __fadd_rn(product, kMagic);
    const float nearest = __fsub_rn(shifted, kMagic);
    worst = fmaxf(worst, fabsf(__fsub_rn(product, nearest)));
    bits[i] = __float_as_uint(shifted);
  }
  if (worst > 0.4999f) {
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      packed |= (static_cast<uint32_t>(quantize_value(values[i], scale, FMOE_NUMERICS_TORCHREF)) & 0xffu) << (8 * i);
    }
    return packed;
  }
  // Low byte of each sum = the integer in two's complement.
  return __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
}

__device__ __forceinline__ float quantize_operand(float scale, int numerics) {
  return numerics == FMOE_NUMERICS_NATIVE ? __fdiv_rn(1.0f, scale) : scale;
}

__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, offset));
  return value;
}

__device__ __forceinline__ int warp_sum(int value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
  return value;
}

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
  return value;
}

}  // namespace fmoe
