/*
 * CPU oracle for the routed-expert MoE path.  TEST INFRASTRUCTURE ONLY: nothing in the
 * shipped package links, imports or calls this file; tests, the smoke check and the
 * CPU-baseline leg of the benchmark are its only users.
 *
 * It restates, as plain scalar C, the arithmetic of the reference CPU implementation
 * (paths are relative to the reference project):
 *
 *   route lists          csrc/moe/arm/i8mm_w8a8/kernels.cpp:583-592
 *   row quantiser        csrc/moe/arm/i8mm_w8a8/kernels.cpp:211-228   (numerics = NATIVE)
 *                        tests/test_moe_w8a8.py:40-43                 (numerics = TORCHREF)
 *   exp(-gate)           csrc/moe/arm/i8mm_w8a8/kernels.cpp:200-209   (FEXPA evaluator)
 *   gate_up epilogue     csrc/moe/arm/i8mm_w8a8/kernels.cpp:230-246 ; tests/test_moe_w8a8.py:61-64
 *   down store           csrc/moe/arm/i8mm_w8a8/kernels.cpp:248-257 ; tests/test_moe_w8a8.py:66
 *   W8A8 top-k merge     csrc/moe/arm/i8mm_w8a8/kernels.cpp:675-688
 *   BF16 expert FFN      src/fused_cpp/moe/naive.py:223-269 ; csrc/moe/arm/sve_bf16/packing.cpp:51-73
 *   BF16 top-k merge     csrc/moe/arm/sve_bf16/route_merge.cpp:48-86
 *   dense W8A8 linear    csrc/i8gemm.cpp:366-399 (scalar fallback)
 *   W8A16 expert FFN     csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:4916-4948, 8740-8760 (int8 weights, bf16
 *                        activations, channel scale on the fp32 accumulator); the variant with the activations as
 *                        16-bit fixed point per row is the CUDA library's own default form, restated here so that it
 *                        can be checked bit for bit, and pinned to the reference to tolerance only
 *
 * Parity pins: tests/golden holds outputs of the reference's own Python functions
 * (tests/test_moe_w8a8.py::_quantize_row/_reference and fused_cpp.moe.naive.fused_moe_naive)
 * on seeded inputs; tests/test_oracle_golden.py checks this file against them.  The native
 * AArch64 kernels cannot run on an x86 host, so NATIVE numerics are pinned only through the
 * shared stages and by reading; that mode is "parity unpinned" against Arm silicon.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fno-fast-math -shared -fPIC (see oracle/build.py).
 * -ffp-contract=off matters: every multiply-add that the reference fuses is written as fmaf()
 * here and every one it does not fuse must stay unfused.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define FMOE_NUMERICS_TORCHREF 0
#define FMOE_NUMERICS_NATIVE 1

/* fp32(2^(i/64)), i = 0..63: the significand table the FEXPA instruction indexes with the
 * low six bits of its operand. */
static const uint32_t k_exp2_table[64] = {
    0x3f800000u, 0x3f8164d2u, 0x3f82cd87u, 0x3f843a29u, 0x3f85aac3u, 0x3f871f62u, 0x3f88980fu, 0x3f8a14d5u,
    0x3f8b95c2u, 0x3f8d1adfu, 0x3f8ea43au, 0x3f9031dcu, 0x3f91c3d3u, 0x3f935a2bu, 0x3f94f4f0u, 0x3f96942du,
    0x3f9837f0u, 0x3f99e046u, 0x3f9b8d3au, 0x3f9d3edau, 0x3f9ef532u, 0x3fa0b051u, 0x3fa27043u, 0x3fa43516u,
    0x3fa5fed7u, 0x3fa7cd94u, 0x3fa9a15bu, 0x3fab7a3au, 0x3fad583fu, 0x3faf3b79u, 0x3fb123f6u, 0x3fb311c4u,
    0x3fb504f3u, 0x3fb6fd92u, 0x3fb8fbafu, 0x3fbaff5bu, 0x3fbd08a4u, 0x3fbf179au, 0x3fc12c4du, 0x3fc346cdu,
    0x3fc5672au, 0x3fc78d75u, 0x3fc9b9beu, 0x3fcbec15u, 0x3fce248cu, 0x3fd06334u, 0x3fd2a81eu, 0x3fd4f35bu,
    0x3fd744fdu, 0x3fd99d16u, 0x3fdbfbb8u, 0x3fde60f5u, 0x3fe0ccdfu, 0x3fe33f89u, 0x3fe5b907u, 0x3fe8396au,
    0x3feac0c7u, 0x3fed4f30u, 0x3fefe4bau, 0x3ff28177u, 0x3ff5257du, 0x3ff7d0dfu, 0x3ffa83b3u, 0x3ffd3e0cu,
};

static inline float bits_to_f32(uint32_t bits) {
  float value;
  memcpy(&value, &bits, 4);
  return value;
}

static inline uint32_t f32_to_bits(float value) {
  uint32_t bits;
  memcpy(&bits, &value, 4);
  return bits;
}

static inline float bf16_to_f32(uint16_t bits) { return bits_to_f32((uint32_t)bits << 16); }

/* store_bf16, kernels.cpp:194-198: add 0x7fff + lsb, keep the high half (nearest-even). */
uint16_t fmoe_oracle_f32_to_bf16(float value) {
  const uint32_t bits = f32_to_bits(value);
  const uint32_t lsb = (bits >> 16) & 1u;
  return (uint16_t)((bits + 0x7fffu + lsb) >> 16);
}

/* exp_fexpa_neg, kernels.cpp:200-209.  FEXPA(bits): exponent field = bits[13:6], fraction =
 * table[bits[5:0]]. */
float fmoe_oracle_expneg(float gate) {
  float x = -gate;
  x = fminf(x, 87.0f);
  x = fmaxf(x, -87.0f);
  const float encoded = fmaf(x, 1.4426950216293335f, 196735.0f);
  const float k = encoded - 196735.0f;
  float residual = fmaf(-k, 0.693145751953125f, x);
  residual = fmaf(-k, 1.428606765330187e-06f, residual);
  const uint32_t enc_bits = f32_to_bits(encoded);
  const uint32_t scale_bits = (((enc_bits >> 6) & 0xffu) << 23) | (k_exp2_table[enc_bits & 63u] & 0x007fffffu);
  const float scale = bits_to_f32(scale_bits);
  const float polynomial = fmaf(residual, 0.5000003576278687f, 1.000003695487976f);
  return fmaf(scale, polynomial * residual, scale);
}

/* Clamped SwiGLU on dequantised gate/up, kernels.cpp:240-244.  limit <= 0 disables the clamp
 * (BF16 path without swiglu_limit). */
static inline uint16_t swiglu_to_bf16(float gate, float up, float limit) {
  if (limit > 0.0f) {
    gate = fminf(gate, limit);
    up = fmaxf(fminf(up, limit), -limit);
  }
  const float value = (gate * up) / (fmoe_oracle_expneg(gate) + 1.0f);
  return fmoe_oracle_f32_to_bf16(value);
}

static inline float round_half_away(float value) {
  /* svrinta: ties away from zero, which is C's roundf. */
  return roundf(value);
}

/* One row of bf16 -> int8 + scale. */
static void quantize_row(const uint16_t* source, int columns, int numerics, int8_t* destination, float* scale_out) {
  float maximum = 0.0f;
  for (int column = 0; column < columns; ++column) {
    maximum = fmaxf(maximum, fabsf(bf16_to_f32(source[column])));
  }
  if (numerics == FMOE_NUMERICS_NATIVE) {
    /* kernels.cpp:219-226 */
    const float scale = maximum > 0.0f ? maximum / 127.0f : 1.0f;
    const float inverse = 1.0f / scale;
    *scale_out = scale;
    for (int column = 0; column < columns; ++column) {
      float value = bf16_to_f32(source[column]) * inverse;
      value = fmaxf(fminf(value, 127.0f), -127.0f);
      destination[column] = (int8_t)round_half_away(value);
    }
  } else {
    /* tests/test_moe_w8a8.py:40-43: scale = max(amax/127, 1e-30); (row/scale).round().clamp(-127,127) */
    float scale = maximum / 127.0f;
    if (scale < 1.0e-30f) scale = 1.0e-30f;
    *scale_out = scale;
    for (int column = 0; column < columns; ++column) {
      float value = rintf(bf16_to_f32(source[column]) / scale); /* rintf: ties to even in the default mode */
      value = fmaxf(fminf(value, 127.0f), -127.0f);
      destination[column] = (int8_t)value;
    }
  }
}

void fmoe_oracle_quantize_rows(const uint16_t* source, int64_t rows, int columns, int numerics, int8_t* destination,
                               float* scales) {
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < rows; ++row) {
    quantize_row(source + row * columns, columns, numerics, destination + row * columns, scales + row);
  }
}

static inline float dequantize(int32_t accumulator, float activation_scale, float channel_scale, int numerics) {
  if (numerics == FMOE_NUMERICS_NATIVE) {
    return (float)accumulator * (activation_scale * channel_scale); /* kernels.cpp:238, 255 */
  }
  return ((float)accumulator * activation_scale) * channel_scale; /* tests/test_moe_w8a8.py:61, 66 */
}

/* Route lists: per expert, flat route ids t*K+slot in ascending order (a stable counting
 * sort by expert id).  Returns -1 if an id is outside [0, experts). */
int fmoe_oracle_route_build(const int64_t* topk_ids, int64_t routes, int experts, int32_t* counts, int32_t* offsets,
                            int32_t* sorted_routes) {
  memset(counts, 0, sizeof(int32_t) * (size_t)experts);
  for (int64_t route = 0; route < routes; ++route) {
    if (topk_ids[route] < 0 || topk_ids[route] >= experts) return -1;
    counts[topk_ids[route]] += 1;
  }
  offsets[0] = 0;
  for (int expert = 0; expert < experts; ++expert) offsets[expert + 1] = offsets[expert] + counts[expert];
  int32_t* cursor = (int32_t*)malloc(sizeof(int32_t) * (size_t)(experts > 0 ? experts : 1));
  memcpy(cursor, offsets, sizeof(int32_t) * (size_t)experts);
  for (int64_t route = 0; route < routes; ++route) sorted_routes[cursor[topk_ids[route]]++] = (int32_t)route;
  free(cursor);
  return 0;
}

static inline int32_t dot_i8(const int8_t* a, const int8_t* b, int n) {
  int32_t sum = 0;
  for (int i = 0; i < n; ++i) sum += (int32_t)a[i] * (int32_t)b[i];
  return sum;
}

/*
 * W8A8 routed-expert forward.  Layouts: x[T,H] bf16; w13[E,2I,H] int8 (gate rows then up rows);
 * s13[E,2I]; w2[E,H,I] int8; s2[E,H]; topk_w[T,K] f32; topk_ids[T,K] i64; out[T,H] bf16.
 * Optional dumps (NULL to skip) are indexed by token (xq, a) or by flat route id t*K+slot.
 */
int fmoe_oracle_w8a8_forward(const uint16_t* x, const int8_t* w13, const float* s13, const int8_t* w2, const float* s2,
                             const float* topk_w, const int64_t* topk_ids, int64_t tokens, int top_k, int experts,
                             int hidden, int inter, int numerics, uint16_t* out, int8_t* dump_xq, float* dump_a,
                             int32_t* dump_acc1, uint16_t* dump_y, int8_t* dump_yq, float* dump_a2,
                             int32_t* dump_acc2, float* dump_route_out) {
  const int64_t routes = tokens * top_k;
  for (int64_t route = 0; route < routes; ++route) {
    if (topk_ids[route] < 0 || topk_ids[route] >= experts) return -1;
  }
  int8_t* xq = (int8_t*)malloc((size_t)(tokens > 0 ? tokens : 1) * hidden);
  float* a = (float*)malloc(sizeof(float) * (size_t)(tokens > 0 ? tokens : 1));
  float* route_out = dump_route_out ? dump_route_out : (float*)malloc(sizeof(float) * (size_t)(routes > 0 ? routes : 1) * hidden);
  /* The reference quantises x[token] once per route; the result only depends on the token. */
  fmoe_oracle_quantize_rows(x, tokens, hidden, numerics, xq, a);
  if (dump_xq) memcpy(dump_xq, xq, (size_t)tokens * hidden);
  if (dump_a) memcpy(dump_a, a, sizeof(float) * (size_t)tokens);

#pragma omp parallel
  {
    int32_t* acc1 = (int32_t*)malloc(sizeof(int32_t) * 2 * (size_t)inter);
    uint16_t* y = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)inter);
    int8_t* yq = (int8_t*)malloc((size_t)inter);
#pragma omp for schedule(dynamic, 1)
    for (int64_t route = 0; route < routes; ++route) {
      const int64_t token = route / top_k;
      const int64_t expert = topk_ids[route];
      const int8_t* xrow = xq + token * hidden;
      const int8_t* w13_e = w13 + expert * 2 * (int64_t)inter * hidden;
      const float* s13_e = s13 + expert * 2 * (int64_t)inter;
      for (int n = 0; n < 2 * inter; ++n) acc1[n] = dot_i8(xrow, w13_e + (int64_t)n * hidden, hidden);
      for (int j = 0; j < inter; ++j) {
        const float gate = dequantize(acc1[j], a[token], s13_e[j], numerics);
        const float up = dequantize(acc1[inter + j], a[token], s13_e[inter + j], numerics);
        y[j] = swiglu_to_bf16(gate, up, 10.0f);
      }
      float a2;
      quantize_row(y, inter, numerics, yq, &a2);
      const int8_t* w2_e = w2 + expert * (int64_t)hidden * inter;
      const float* s2_e = s2 + expert * (int64_t)hidden;
      float* route_row = route_out + route * hidden;
      for (int h = 0; h < hidden; ++h) {
        const int32_t acc2 = dot_i8(yq, w2_e + (int64_t)h * inter, inter);
        if (dump_acc2) dump_acc2[route * hidden + h] = acc2;
        route_row[h] = dequantize(acc2, a2, s2_e[h], numerics);
      }
      if (dump_acc1) memcpy(dump_acc1 + route * 2 * inter, acc1, sizeof(int32_t) * 2 * (size_t)inter);
      if (dump_y) memcpy(dump_y + route * inter, y, sizeof(uint16_t) * (size_t)inter);
      if (dump_yq) memcpy(dump_yq + route * inter, yq, (size_t)inter);
      if (dump_a2) dump_a2[route] = a2;
    }
    free(acc1);
    free(y);
    free(yq);
  }

  /* kernels.cpp:675-688: fused multiply-add chain in slot order, starting from zero. */
#pragma omp parallel for schedule(static)
  for (int64_t token = 0; token < tokens; ++token) {
    for (int h = 0; h < hidden; ++h) {
      float accumulator = 0.0f;
      for (int slot = 0; slot < top_k; ++slot) {
        const int64_t route = token * top_k + slot;
        accumulator = fmaf(route_out[route * hidden + h], topk_w[route], accumulator);
      }
      out[token * hidden + h] = fmoe_oracle_f32_to_bf16(accumulator);
    }
  }
  free(xq);
  free(a);
  if (!dump_route_out) free(route_out);
  return 0;
}

/*
 * Expert-side half of the W8A8 forward for rows that are already quantised (one route per row):
 * gate_up dot products, dequant + clamp-10 SwiGLU + bf16, requantise, down dot products, dequant.
 * Same statements as the per-route loop of fmoe_oracle_w8a8_forward (kernels.cpp:646-671); used to
 * check the expert-parallel split, where quantisation and GEMMs run on different ranks.
 */
int fmoe_oracle_w8a8_route_rows(const int8_t* rows_q, const float* rows_scale, const int64_t* rows_expert, int64_t rows,
                                const int8_t* w13, const float* s13, const int8_t* w2, const float* s2, int experts,
                                int hidden, int inter, int numerics, float* route_out) {
  for (int64_t row = 0; row < rows; ++row) {
    if (rows_expert[row] < 0 || rows_expert[row] >= experts) return -1;
  }
#pragma omp parallel
  {
    int32_t* acc1 = (int32_t*)malloc(sizeof(int32_t) * 2 * (size_t)inter);
    uint16_t* y = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)inter);
    int8_t* yq = (int8_t*)malloc((size_t)inter);
#pragma omp for schedule(dynamic, 1)
    for (int64_t row = 0; row < rows; ++row) {
      const int64_t expert = rows_expert[row];
      const int8_t* xrow = rows_q + row * hidden;
      const int8_t* w13_e = w13 + expert * 2 * (int64_t)inter * hidden;
      const float* s13_e = s13 + expert * 2 * (int64_t)inter;
      for (int n = 0; n < 2 * inter; ++n) acc1[n] = dot_i8(xrow, w13_e + (int64_t)n * hidden, hidden);
      for (int j = 0; j < inter; ++j) {
        const float gate = dequantize(acc1[j], rows_scale[row], s13_e[j], numerics);
        const float up = dequantize(acc1[inter + j], rows_scale[row], s13_e[inter + j], numerics);
        y[j] = swiglu_to_bf16(gate, up, 10.0f);
      }
      float a2;
      quantize_row(y, inter, numerics, yq, &a2);
      const int8_t* w2_e = w2 + expert * (int64_t)hidden * inter;
      const float* s2_e = s2 + expert * (int64_t)hidden;
      for (int h = 0; h < hidden; ++h) {
        route_out[row * hidden + h] = dequantize(dot_i8(yq, w2_e + (int64_t)h * inter, inter), a2, s2_e[h], numerics);
      }
    }
    free(acc1);
    free(y);
    free(yq);
  }
  return 0;
}

/* W8A8 merge alone (kernels.cpp:675-688): fused chain in slot order from zero, bf16 store. */
void fmoe_oracle_merge_w8a8_path(const float* route_out, const float* topk_w, int64_t tokens, int top_k, int hidden,
                                 uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t token = 0; token < tokens; ++token) {
    for (int h = 0; h < hidden; ++h) {
      float accumulator = 0.0f;
      for (int slot = 0; slot < top_k; ++slot) {
        const int64_t route = token * top_k + slot;
        accumulator = fmaf(route_out[route * hidden + h], topk_w[route], accumulator);
      }
      out[token * hidden + h] = fmoe_oracle_f32_to_bf16(accumulator);
    }
  }
}

/* route_merge.cpp:48-69: split at the largest power of two below count; leaves are w*route. */
static float merge_tree(const float* route_out, const float* weights, int64_t hidden, int h, int begin, int count) {
  if (count == 1) return route_out[(int64_t)begin * hidden + h] * weights[begin];
  int left = 1;
  while ((left << 1) < count) left <<= 1;
  const float lhs = merge_tree(route_out, weights, hidden, h, begin, left);
  const float rhs = merge_tree(route_out, weights, hidden, h, begin + left, count - left);
  return lhs + rhs;
}

/* BF16 top-k merge: pairwise tree for K in {2,4,6,8}, sequential fused chain otherwise
 * (route_merge.cpp:78-86, 144-163). */
void fmoe_oracle_merge_bf16_path(const float* route_out, const float* topk_w, int64_t tokens, int top_k, int hidden,
                                 uint16_t* out) {
  const int fixed = top_k == 2 || top_k == 4 || top_k == 6 || top_k == 8;
#pragma omp parallel for schedule(static)
  for (int64_t token = 0; token < tokens; ++token) {
    const float* token_routes = route_out + token * top_k * hidden;
    const float* weights = topk_w + token * top_k;
    for (int h = 0; h < hidden; ++h) {
      float value;
      if (fixed) {
        value = merge_tree(token_routes, weights, hidden, h, 0, top_k);
      } else {
        value = 0.0f;
        for (int slot = 0; slot < top_k; ++slot) value = fmaf(token_routes[(int64_t)slot * hidden + h], weights[slot], value);
      }
      out[token * hidden + h] = fmoe_oracle_f32_to_bf16(value);
    }
  }
}

static inline float dot_bf16(const uint16_t* a, const uint16_t* b, int n) {
  /* fp32 accumulation of exact bf16 products; summation order is not part of the contract
   * (the tolerance for BF16 outputs covers it).  Eight partial sums keep the loop vectorisable. */
  float partial[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int i = 0;
  for (; i + 8 <= n; i += 8) {
    for (int lane = 0; lane < 8; ++lane) partial[lane] += bf16_to_f32(a[i + lane]) * bf16_to_f32(b[i + lane]);
  }
  float sum = ((partial[0] + partial[1]) + (partial[2] + partial[3])) + ((partial[4] + partial[5]) + (partial[6] + partial[7]));
  for (; i < n; ++i) sum += bf16_to_f32(a[i]) * bf16_to_f32(b[i]);
  return sum;
}

/*
 * The other gated activations of the BF16 op (activation_to_bf16, csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:1911-1936;
 * arithmetic as in src/fused_cpp/moe/naive.py:28-54): 2 = gelu(erf)(gate) * up, 3 = swigluoai
 * ((clamp(up, +-7) + 1) * g * sigmoid(1.702 g), g = min(gate, 7)).  Compared to tolerance, so libm's erff / expf serve.
 */
static inline uint16_t other_activation_to_bf16(int activation, float gate, float up) {
  float value;
  if (activation == 2) {
    value = 0.5f * gate * (1.0f + erff(gate * 0.70710678118654752440f)) * up;
  } else {
    gate = gate < 7.0f ? gate : 7.0f;
    up = up > 7.0f ? 7.0f : (up < -7.0f ? -7.0f : up);
    value = (up + 1.0f) * (gate / (1.0f + expf(-1.702f * gate)));
  }
  return fmoe_oracle_f32_to_bf16(value);
}

/*
 * BF16 routed-expert forward: bf16 operands, fp32 accumulation, gated activation rounded to bf16,
 * fp32 route rows, tree/chain merge.  activation 0: SiLU(gate)*up with swiglu_limit <= 0 plain, 10 the clamp-10
 * variant; 2, 3: see above.  w13_bias[E, 2I] / w2_bias[E, H] (fp32, NULL = none) are added to the accumulators
 * before the activation / before the merge (fused_moe_bf16_tiled.cpp:6420-6427; F.linear(..., bias) in naive.py:229-239).
 */
int fmoe_oracle_bf16_forward_ex(const uint16_t* x, const uint16_t* w13, const uint16_t* w2, const float* topk_w,
                                const int64_t* topk_ids, int64_t tokens, int top_k, int experts, int hidden, int inter,
                                float swiglu_limit, int activation, const float* w13_bias, const float* w2_bias,
                                uint16_t* out, uint16_t* dump_y, float* dump_route_out);

int fmoe_oracle_bf16_forward(const uint16_t* x, const uint16_t* w13, const uint16_t* w2, const float* topk_w,
                             const int64_t* topk_ids, int64_t tokens, int top_k, int experts, int hidden, int inter,
                             float swiglu_limit, uint16_t* out, uint16_t* dump_y, float* dump_route_out) {
  return fmoe_oracle_bf16_forward_ex(x, w13, w2, topk_w, topk_ids, tokens, top_k, experts, hidden, inter, swiglu_limit, 0, NULL,
                                     NULL, out, dump_y, dump_route_out);
}

int fmoe_oracle_bf16_forward_ex(const uint16_t* x, const uint16_t* w13, const uint16_t* w2, const float* topk_w,
                                const int64_t* topk_ids, int64_t tokens, int top_k, int experts, int hidden, int inter,
                                float swiglu_limit, int activation, const float* w13_bias, const float* w2_bias,
                                uint16_t* out, uint16_t* dump_y, float* dump_route_out) {
  const int64_t routes = tokens * top_k;
  for (int64_t route = 0; route < routes; ++route) {
    if (topk_ids[route] < 0 || topk_ids[route] >= experts) return -1;
  }
  float* route_out = dump_route_out ? dump_route_out : (float*)malloc(sizeof(float) * (size_t)(routes > 0 ? routes : 1) * hidden);
#pragma omp parallel
  {
    uint16_t* y = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)inter);
#pragma omp for schedule(dynamic, 1)
    for (int64_t route = 0; route < routes; ++route) {
      const int64_t token = route / top_k;
      const int64_t expert = topk_ids[route];
      const uint16_t* xrow = x + token * hidden;
      const uint16_t* w13_e = w13 + expert * 2 * (int64_t)inter * hidden;
      const float* b13 = w13_bias ? w13_bias + expert * 2 * (int64_t)inter : NULL;
      const float* b2 = w2_bias ? w2_bias + expert * (int64_t)hidden : NULL;
      for (int j = 0; j < inter; ++j) {
        float gate = dot_bf16(xrow, w13_e + (int64_t)j * hidden, hidden);
        float up = dot_bf16(xrow, w13_e + (int64_t)(inter + j) * hidden, hidden);
        if (b13) {
          gate += b13[j];
          up += b13[inter + j];
        }
        y[j] = activation == 0 ? swiglu_to_bf16(gate, up, swiglu_limit) : other_activation_to_bf16(activation, gate, up);
      }
      const uint16_t* w2_e = w2 + expert * (int64_t)hidden * inter;
      for (int h = 0; h < hidden; ++h) {
        const float value = dot_bf16(y, w2_e + (int64_t)h * inter, inter);
        route_out[route * hidden + h] = b2 ? value + b2[h] : value;
      }
      if (dump_y) memcpy(dump_y + route * inter, y, sizeof(uint16_t) * (size_t)inter);
    }
    free(y);
  }
  fmoe_oracle_merge_bf16_path(route_out, topk_w, tokens, top_k, hidden, out);
  if (!dump_route_out) free(route_out);
  return 0;
}

static inline float dot_bf16_i8(const uint16_t* a, const int8_t* b, int n) {
  /* bf16 x int8 products are exact in fp32 (8 + 7 significant bits); summation order is covered by the tolerance. */
  float partial[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int i = 0;
  for (; i + 8 <= n; i += 8) {
    for (int lane = 0; lane < 8; ++lane) partial[lane] += bf16_to_f32(a[i + lane]) * (float)b[i + lane];
  }
  float sum = ((partial[0] + partial[1]) + (partial[2] + partial[3])) + ((partial[4] + partial[5]) + (partial[6] + partial[7]));
  for (; i < n; ++i) sum += bf16_to_f32(a[i]) * (float)b[i];
  return sum;
}

/*
 * W8A16 routed-expert forward: int8 weights with per-output-channel fp32 scales, bf16 activations that are not
 * quantised.  acc = sum_k x[k] * q[n,k] in fp32, value = acc * scale[n] (the reference applies the packed
 * per-channel scales to its accumulators, csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:4916-4948, 8740-8760), then
 * the BF16 path: activation rounded to bf16, fp32 route rows, tree / chain merge.
 */
int fmoe_oracle_w8a16_forward(const uint16_t* x, const int8_t* w13, const float* s13, const int8_t* w2, const float* s2,
                              const float* topk_w, const int64_t* topk_ids, int64_t tokens, int top_k, int experts,
                              int hidden, int inter, float swiglu_limit, int activation, uint16_t* out, uint16_t* dump_y,
                              float* dump_route_out) {
  const int64_t routes = tokens * top_k;
  for (int64_t route = 0; route < routes; ++route) {
    if (topk_ids[route] < 0 || topk_ids[route] >= experts) return -1;
  }
  float* route_out = dump_route_out ? dump_route_out : (float*)malloc(sizeof(float) * (size_t)(routes > 0 ? routes : 1) * hidden);
#pragma omp parallel
  {
    uint16_t* y = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)inter);
#pragma omp for schedule(dynamic, 1)
    for (int64_t route = 0; route < routes; ++route) {
      const int64_t token = route / top_k;
      const int64_t expert = topk_ids[route];
      const uint16_t* xrow = x + token * hidden;
      const int8_t* w13_e = w13 + expert * 2 * (int64_t)inter * hidden;
      const float* s13_e = s13 + expert * 2 * (int64_t)inter;
      for (int j = 0; j < inter; ++j) {
        const float gate = dot_bf16_i8(xrow, w13_e + (int64_t)j * hidden, hidden) * s13_e[j];
        const float up = dot_bf16_i8(xrow, w13_e + (int64_t)(inter + j) * hidden, hidden) * s13_e[inter + j];
        y[j] = activation == 0 ? swiglu_to_bf16(gate, up, swiglu_limit) : other_activation_to_bf16(activation, gate, up);
      }
      const int8_t* w2_e = w2 + expert * (int64_t)hidden * inter;
      const float* s2_e = s2 + expert * (int64_t)hidden;
      for (int h = 0; h < hidden; ++h) route_out[route * hidden + h] = dot_bf16_i8(y, w2_e + (int64_t)h * inter, inter) * s2_e[h];
      if (dump_y) memcpy(dump_y + route * inter, y, sizeof(uint16_t) * (size_t)inter);
    }
    free(y);
  }
  fmoe_oracle_merge_bf16_path(route_out, topk_w, tokens, top_k, hidden, out);
  if (!dump_route_out) free(route_out);
  return 0;
}

/*
 * W8A16 with the activations carried as 16-bit fixed point per row (the form the CUDA library runs by default; not a
 * statement of the reference, whose W8A16 kernels keep bf16 activations - it is pinned to the reference only through
 * the tolerance against fmoe_oracle_w8a16_forward and the fused_moe_naive golden outputs).  Per row:
 * a = amax / 32512 (1 for an all-zero row), X[k] = clamp(rint(x[k] / a), +-32512); the integer dot product
 * sum_k X[k] * q[n,k] is exact (int64), rounded to fp32 once, value = (fp32(dot) * a) * scale[n]; then the BF16 path
 * (activation to bf16, the same fixed-point step on the intermediate row, fp32 route rows, tree / chain merge).
 */
static float fixed_point_row(const uint16_t* row, int n, int32_t* fixed) {
  float maximum = 0.0f;
  for (int i = 0; i < n; ++i) maximum = fmaxf(maximum, fabsf(bf16_to_f32(row[i])));
  const float scale = maximum > 0.0f ? maximum / 32512.0f : 1.0f;
  for (int i = 0; i < n; ++i) {
    float value = rintf(bf16_to_f32(row[i]) / scale);
    value = fmaxf(fminf(value, 32512.0f), -32512.0f);
    fixed[i] = (int32_t)value;
  }
  return scale;
}

static inline float dot_fixed_i8(const int32_t* a, const int8_t* b, int n) {
  int64_t sum = 0;
  for (int i = 0; i < n; ++i) sum += (int64_t)a[i] * (int64_t)b[i];
  return (float)sum; /* one rounding, to nearest even */
}

int fmoe_oracle_w8a16_fixed_forward(const uint16_t* x, const int8_t* w13, const float* s13, const int8_t* w2, const float* s2,
                                    const float* topk_w, const int64_t* topk_ids, int64_t tokens, int top_k, int experts,
                                    int hidden, int inter, float swiglu_limit, int activation, uint16_t* out, uint16_t* dump_y,
                                    float* dump_route_out) {
  const int64_t routes = tokens * top_k;
  for (int64_t route = 0; route < routes; ++route) {
    if (topk_ids[route] < 0 || topk_ids[route] >= experts) return -1;
  }
  float* route_out = dump_route_out ? dump_route_out : (float*)malloc(sizeof(float) * (size_t)(routes > 0 ? routes : 1) * hidden);
#pragma omp parallel
  {
    uint16_t* y = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)inter);
    int32_t* fixed = (int32_t*)malloc(sizeof(int32_t) * (size_t)(hidden > inter ? hidden : inter));
#pragma omp for schedule(dynamic, 1)
    for (int64_t route = 0; route < routes; ++route) {
      const int64_t token = route / top_k;
      const int64_t expert = topk_ids[route];
      const float a = fixed_point_row(x + token * hidden, hidden, fixed);
      const int8_t* w13_e = w13 + expert * 2 * (int64_t)inter * hidden;
      const float* s13_e = s13 + expert * 2 * (int64_t)inter;
      for (int j = 0; j < inter; ++j) {
        const float gate = (dot_fixed_i8(fixed, w13_e + (int64_t)j * hidden, hidden) * a) * s13_e[j];
        const float up = (dot_fixed_i8(fixed, w13_e + (int64_t)(inter + j) * hidden, hidden) * a) * s13_e[inter + j];
        y[j] = activation == 0 ? swiglu_to_bf16(gate, up, swiglu_limit) : other_activation_to_bf16(activation, gate, up);
      }
      const float a2 = fixed_point_row(y, inter, fixed);
      const int8_t* w2_e = w2 + expert * (int64_t)hidden * inter;
      const float* s2_e = s2 + expert * (int64_t)hidden;
      for (int h = 0; h < hidden; ++h) route_out[route * hidden + h] = (dot_fixed_i8(fixed, w2_e + (int64_t)h * inter, inter) * a2) * s2_e[h];
      if (dump_y) memcpy(dump_y + route * inter, y, sizeof(uint16_t) * (size_t)inter);
    }
    free(y);
    free(fixed);
  }
  fmoe_oracle_merge_bf16_path(route_out, topk_w, tokens, top_k, hidden, out);
  if (!dump_route_out) free(route_out);
  return 0;
}

/*
 * Dense dynamic-quant W8A8 linear, scalar fallback of csrc/i8gemm.cpp:366-399: per-row
 * scale = amax/127 (1 when the row is zero), q = clamp(nearbyint(x/scale), -128, 127),
 * out = (acc * x_scale) * w_scale[n] (+ bias).  x is fp32 here (bf16 callers widen first).
 * out_bf16 != 0 stores bf16 (nearest-even), else fp32.
 */
void fmoe_oracle_i8gemm_dynamic(const float* x, int64_t rows, int k, const int8_t* weight, const float* weight_scale,
                                int n, const float* bias, void* out, int out_bf16, int clamp_low) {
#pragma omp parallel
  {
    int8_t* q = (int8_t*)malloc((size_t)k);
#pragma omp for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
      const float* xrow = x + row * k;
      float maximum = 0.0f;
      for (int i = 0; i < k; ++i) maximum = fmaxf(maximum, fabsf(xrow[i]));
      const float scale = maximum > 0.0f ? maximum / 127.0f : 1.0f;
      for (int i = 0; i < k; ++i) {
        float value = rintf(xrow[i] / scale);
        value = fmaxf(fminf(value, 127.0f), (float)clamp_low); /* -128 single GEMM (:395), -127 paired (:505) */
        q[i] = (int8_t)value;
      }
      for (int column = 0; column < n; ++column) {
        const int32_t acc = dot_i8(q, weight + (int64_t)column * k, k);
        float value = ((float)acc * scale) * weight_scale[column];
        if (bias) value += bias[column];
        if (out_bf16) {
          ((uint16_t*)out)[row * n + column] = fmoe_oracle_f32_to_bf16(value);
        } else {
          ((float*)out)[row * n + column] = value;
        }
      }
    }
    free(q);
  }
}
