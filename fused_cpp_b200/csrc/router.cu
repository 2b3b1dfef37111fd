// Router front-end: scores -> top-k -> renormalised routing weights, the step that precedes the routed-expert
// path.  The reference receives topk_weights / topk_ids from its caller (src/fused_cpp/moe/naive.py:4-7;
// vLLM computes them); the arithmetic restated here is the one the benchmark configurations name: softmax over the
// expert logits, top-k, weights renormalised to sum to one, optionally scaled, and the sigmoid-with-selection-bias
// variant of DeepSeek-V3 routers.  The outputs have the types the path takes (fp32 weights, int64 ids), so the ids
// never leave the GPU between the router and the route build.
//
// One warp per token.  Lane l holds logits l, l+32, ...; the row maximum and the softmax denominator are shuffle
// reductions; the top-k is k rounds of a warp arg-max over the values not yet taken (ties go to the lower expert
// id, so the result is a function of the logits alone).
#include "common.cuh"
#include "kernels.h"

namespace fmoe {

namespace {

constexpr int kRouterWarps = 4;
constexpr int kRouterMaxPerLane = 64;  // experts <= 2048

__device__ __forceinline__ void warp_argmax(float& value, int& index) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float other_value = __shfl_xor_sync(0xffffffffu, value, offset);
    const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
    if (other_value > value || (other_value == value && other_index < index)) {
      value = other_value;
      index = other_index;
    }
  }
}

template <int kPerLane>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ selection_bias, int64_t tokens, int experts, int top_k,
                   int sigmoid, int renormalize, float scaling, float* __restrict__ topk_weights, int64_t* __restrict__ topk_ids) {
  const int lane = threadIdx.x & 31;
  const int64_t token = static_cast<int64_t>(blockIdx.x) * kRouterWarps + (threadIdx.x >> 5);
  if (token >= tokens) return;
  const float* row = logits + token * experts;
  float score[kPerLane];   // what the weights are made of
  // What the selection compares.  Without a selection bias that is the logit itself: softmax and sigmoid are
  // monotone, so the top-k of the scores is the top-k of the logits, and comparing logits keeps the choice free of
  // the rounding of exp and of the division (two logits that differ always order the same way).  With a bias the
  // selection compares score + bias.
  float choice[kPerLane];
  float row_max = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    score[i] = e < experts ? row[e] : -INFINITY;
    choice[i] = score[i];
    row_max = fmaxf(row_max, score[i]);
  }
  row_max = warp_max(row_max);
  float denominator = 0.0f;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    if (e < experts) {
      if (sigmoid) {
        score[i] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-score[i])));
      } else {
        score[i] = expf(__fsub_rn(score[i], row_max));
        denominator = __fadd_rn(denominator, score[i]);
      }
      if (selection_bias != nullptr) choice[i] = __fadd_rn(score[i], selection_bias[e]);
    } else {
      score[i] = 0.0f;
      choice[i] = -INFINITY;
    }
  }
  if (!sigmoid) {
    denominator = warp_sum(denominator);
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      score[i] = __fdiv_rn(score[i], denominator);  // the softmax probability
      const int e = lane + 32 * i;
      if (e < experts && selection_bias != nullptr) choice[i] = __fadd_rn(score[i], selection_bias[e]);
    }
  }
  // k rounds of arg-max.  Lane r keeps the r-th winner.
  float kept_weight = 0.0f;
  int kept_id = 0;
  float total = 0.0f;
  for (int round = 0; round < top_k; ++round) {
    float best = -INFINITY;
    int best_index = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int e = lane + 32 * i;
      if (choice[i] > best || (choice[i] == best && e < best_index)) {  // ascending e inside a lane: the lower id wins ties
        best = choice[i];
        best_index = e;
      }
    }
    warp_argmax(best, best_index);
    // The owner hands out the unbiased score and retires the entry.
    float weight = 0.0f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      if (lane + 32 * i == best_index) {
        weight = score[i];
        choice[i] = -INFINITY;
      }
    }
    weight = __shfl_sync(0xffffffffu, weight, best_index & 31);
    total = __fadd_rn(total, weight);
    if (lane == round) {
      kept_weight = weight;
      kept_id = best_index;
    }
  }
  if (lane < top_k) {
    float weight = kept_weight;
    if (renormalize) weight = __fdiv_rn(weight, total);
    weight = __fmul_rn(weight, scaling);
    topk_weights[token * top_k + lane] = weight;
    topk_ids[token * top_k + lane] = kept_id;
  }
}

}  // namespace

cudaError_t launch_router_topk(const float* logits, const float* selection_bias, int64_t tokens, int experts, int top_k, int sigmoid,
                               int renormalize, float scaling, float* topk_weights, int64_t* topk_ids, cudaStream_t stream) {
  if (tokens <= 0) return cudaSuccess;
  const unsigned blocks = static_cast<unsigned>((tokens + kRouterWarps - 1) / kRouterWarps);
  const int per_lane = (experts + 31) / 32;
#define FMOE_ROUTER_CASE(n)                                                                                                    \
  if (per_lane <= n) {                                                                                                         \
    router_topk_kernel<n><<<blocks, kRouterWarps * 32, 0, stream>>>(logits, selection_bias, tokens, experts, top_k, sigmoid,   \
                                                                     renormalize, scaling, topk_weights, topk_ids);            \
    return cudaGetLastError();                                                                                                 \
  }
  FMOE_ROUTER_CASE(1)
  FMOE_ROUTER_CASE(2)
  FMOE_ROUTER_CASE(4)
  FMOE_ROUTER_CASE(8)
  FMOE_ROUTER_CASE(16)
  FMOE_ROUTER_CASE(32)
  FMOE_ROUTER_CASE(kRouterMaxPerLane)
#undef FMOE_ROUTER_CASE
  return cudaErrorInvalidValue;
}

}  // namespace fmoe
