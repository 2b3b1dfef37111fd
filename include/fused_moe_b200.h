/*
 * C ABI of the B200 routed-expert MoE library (libfused_moe_b200.so).
 *
 * The reference project has no C ABI of its own: its boundary for this path is two pybind11 torch
 * extensions (fused_cpp._moe_C, csrc/moe/module.cpp:10-264, and the i8gemm_* ops of fused_cpp._C,
 * csrc/module.cpp:220-233).  Each entry point below names the reference function whose work it does;
 * the Python package above this ABI (fused_cpp_b200.moe) keeps the reference's op names and
 * argument lists and forwards device pointers here.
 *
 * Conventions
 *   - every data pointer is a DEVICE pointer on the current CUDA device unless a comment says "host";
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); calls are
 *     asynchronous: they enqueue kernels and return, no device-wide synchronisation;
 *   - the library allocates no device memory in the forward calls: the caller passes a workspace of
 *     at least *_workspace_bytes() bytes, 256-byte aligned, private to one call at a time;
 *   - return value: FMOE_OK or an FMOE_ERR_* code; fmoe_last_error() gives the text (thread-local);
 *   - errors that only the device can see (an expert id out of range, a bounded wait that gave up)
 *     are recorded in the workspace status block and read back with fmoe_read_status();
 *   - there is no CPU fallback: on a device that is not compute capability 10.x every call fails
 *     with FMOE_ERR_UNSUPPORTED_DEVICE.
 *
 * Tensor layouts (row-major, innermost last): x[T,H] bf16; topk_weights[T,K] fp32; topk_ids[T,K]
 * int64; W8A8: w13[E,2I,H] int8 (gate rows then up rows), s13[E,2I] fp32, w2[E,H,I] int8, s2[E,H]
 * fp32; BF16: w13[E,2I,H], w2[E,H,I] bf16; out[T,H] bf16.  H and I must be multiples of 16.
 */
#ifndef FUSED_MOE_B200_H_
#define FUSED_MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FMOE_ABI_VERSION 2

#if defined(__GNUC__)
#define FMOE_API __attribute__((visibility("default")))
#else
#define FMOE_API
#endif

#define FMOE_OK 0
#define FMOE_ERR_INVALID_ARGUMENT 1
#define FMOE_ERR_CUDA 2
#define FMOE_ERR_WORKSPACE 3
#define FMOE_ERR_EXPERT_ID_RANGE 4   /* device-detected: a topk id outside [0, E) */
#define FMOE_ERR_DEVICE_WAIT 5       /* device-detected: a bounded barrier wait gave up */
#define FMOE_ERR_UNSUPPORTED_DEVICE 6

/* Which of the reference's two arithmetic statements the W8A8 path follows. */
#define FMOE_NUMERICS_TORCHREF 0 /* tests/test_moe_w8a8.py:40-69: x/scale, ties-to-even, (acc*a)*s */
#define FMOE_NUMERICS_NATIVE 1   /* csrc/moe/arm/i8mm_w8a8/kernels.cpp:211-257: x*(1/scale), ties away, acc*(a*s) */

/* Grouped-GEMM implementation: there is one, on tcgen05 tensor cores.  0 and 2 both select it (2 is kept so that
 * callers written against earlier headers keep working); any other value is refused. */
#define FMOE_GEMM_AUTO 0
#define FMOE_GEMM_UMMA 2

typedef struct fmoe_config {
  int32_t numerics;      /* FMOE_NUMERICS_* (W8A8 only) */
  int32_t gemm_impl;     /* FMOE_GEMM_* */
  int32_t gate_up_tile;  /* rows of one expert per work item in the gate_up GEMM: 16..256, 512 = two-SM pairs of 256 rows; 0 = auto */
  int32_t down_tile;     /* same for the down GEMM; 0 = auto */
  float swiglu_limit;    /* BF16: 0 = plain SiLU, 10 = clamp-10 SwiGLU.  W8A8 requires 10. */
  int32_t activation;    /* BF16 only: FMOE_ACTIVATION_* (W8A8 requires SILU) */
  void* stage_timer;     /* optional handle from fmoe_stage_timer_create: per-stage CUDA events are recorded */
  int32_t* dump_acc1;    /* optional [T*K, 2I] int32 (W8A8) / fp32 (BF16): raw gate_up accumulators, sorted-row order */
  int32_t* dump_acc2;    /* optional [T*K, H]: raw down accumulators, sorted-row order */
  /* BF16 only, optional per-expert biases in fp32 (the reference converts them to fp32 as well,
   * csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:6420-6427): w13_bias[E, 2I] (gate channels then up channels) is added
   * to the gate_up accumulators before the activation, w2_bias[E, H] to every route row before the top-k merge. */
  const float* w13_bias;
  const float* w2_bias;
  /* 1 = compact route rows (opt-in): the down GEMM stores every route's result row as bf16 instead of fp32 and the
   * merge widens them again: half the bytes of the largest intermediate (4*T*K*H written and read at fp32).  The
   * int8 / int32 stages are untouched and stay bit-exact; the bf16 output is then computed from rows rounded to
   * bf16, so it matches the fp32-row result to tolerance (relative L2 <= 5e-3), not bit for bit.  0 (default)
   * keeps the reference's fp32 rows (csrc/moe/arm/i8mm_w8a8/kernels.cpp:248-257; its BF16 path has the same
   * opt-in, FUSED_CPP_MOE_W2_BF16_ROUTE, csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:1016-1019). */
  int32_t route_rows_bf16;
  int32_t w8a16_form;    /* fmoe_w8a16_forward only: FMOE_W8A16_* below */
} fmoe_config;

/* How fmoe_w8a16_forward carries the 16-bit activations to the int8 weights.
 * FIXED_POINT (default): every activation row (and every row of the intermediate) becomes 16-bit fixed point,
 *   X = rint(x / a), a = rowmax / 32512, held as two int8 planes X = 256 * high + low; both planes meet the int8
 *   weights as they lie in HBM on the int8 tensor-core path, the exact integer dot product 256 * acc(high) + acc(low)
 *   is rounded to fp32 once, then multiplied by a and by the channel scale.  |x - a X| <= rowmax * 2^-16: 128 times
 *   finer than one bf16 step at the row maximum; elements below rowmax / 128 lose relative precision, which the
 *   dot product does not see (against the bf16-activation form: relative L2 of 2e-4 on the fp32 route rows of N(0,1)
 *   inputs, most of it bf16 roundings of intermediate elements that fall the other way).
 *   Nothing is widened on the SM, so decode streams the weights at the HBM rate like the W8A8 path.
 * BF16_ACTIVATIONS: the activations stay bf16 bit for bit; the int8 weight tiles are widened to bf16 on the SM after
 *   they crossed HBM as bytes and the product runs on the bf16 tensor-core path with fp32 accumulation.  About half
 *   the decode speed (the widening, not HBM, is the limit). */
#define FMOE_W8A16_FIXED_POINT 0
#define FMOE_W8A16_BF16_ACTIVATIONS 1

/* Gated activations of the BF16 op (activation_to_bf16, csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:1911-1936):
 * SILU = gate * up / (1 + exp(-gate)) with the optional clamp of swiglu_limit; GELU = gelu_erf(gate) * up;
 * SWIGLUOAI = (clamp(up, +-7) + 1) * g * sigmoid(1.702 g) with g = min(gate, 7).  The kernels take gate channels
 * [0, I) and up channels [I, 2I) of w13 for every activation (callers holding the interleaved SWIGLUOAI layout
 * de-interleave once at preparation). */
#define FMOE_ACTIVATION_SILU 0
#define FMOE_ACTIVATION_GELU 2
#define FMOE_ACTIVATION_SWIGLUOAI 3

/* Byte offsets of the regions of a forward workspace (all 256-byte aligned).  Rows of the
 * per-route regions are in SORTED order: position p holds flat route sorted_routes[p]. */
typedef struct fmoe_workspace_layout {
  size_t total_bytes;
  size_t status;         /* int32[16]: [0] error, [1] detail, [2] work items, [3] active experts */
  size_t counts;         /* int32[E]   routes per expert */
  size_t offsets;        /* int32[E+1] exclusive prefix of counts */
  size_t sorted_routes;  /* int32[T*K] flat route ids t*K+slot grouped by expert, ascending inside an expert */
  size_t row_expert;     /* int32[T*K] expert of each sorted row */
  size_t items;          /* int32[4*max_items] (expert, first row, rows, reserved) per work item; two lists */
  size_t scratch;        /* route-build scratch */
  size_t a_rows;         /* W8A8: int8[T*K,H] quantised token rows; BF16: bf16[T*K,H] gathered rows */
  size_t a_scale;        /* W8A8: fp32[T*K] activation scales */
  size_t y;              /* bf16[T*K,I] SiLU(gate)*up */
  size_t yq;             /* W8A8: int8[T*K,I] */
  size_t y_scale;        /* W8A8: fp32[T*K] */
  size_t route_out;      /* fp32[T*K,H], row = FLAT route id (already un-permuted) */
  size_t route_pos;      /* int32[T*K] sorted position of every flat route (-1 = dropped): inverse of sorted_routes */
} fmoe_workspace_layout;

/* ---- library state -------------------------------------------------------------------------- */

FMOE_API int fmoe_abi_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
FMOE_API const char* fmoe_last_error(void);

/* 1 if `device` is a compute-capability-10.x GPU this library can run on, else 0. */
FMOE_API int fmoe_device_supported(int device);

/* Synchronises `stream` and returns the status block of `workspace`: *error is FMOE_OK or the first
 * device-detected error, *detail its argument (e.g. the offending flat route id). */
FMOE_API int fmoe_read_status(const void* workspace, void* stream, int32_t* error, int32_t* detail);

/* ---- per-stage timing ------------------------------------------------------------------------ */

/* Stages of one forward call, in launch order.  With a stage timer in fmoe_config the forward records
 * a CUDA event on its stream before the first stage and after every stage; this is the GPU form of
 * the reference's FUSED_CPP_MOE_STAGE_TIMING report (csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:6756-6762). */
#define FMOE_STAGE_ROUTE 0      /* route build (3 kernels) */
#define FMOE_STAGE_QUANT_IN 1   /* activation quantise + gather (W8A8) / gather (BF16) */
#define FMOE_STAGE_GATE_UP 2    /* grouped gate_up GEMM + SwiGLU epilogue */
#define FMOE_STAGE_QUANT_MID 3  /* intermediate requantise (W8A8; empty for BF16) */
#define FMOE_STAGE_DOWN 4       /* grouped down GEMM + dequant/un-permute epilogue */
#define FMOE_STAGE_MERGE 5      /* top-k merge */
#define FMOE_STAGES 6

/* A timer holds events for up to max_calls forward calls; calls beyond that are not recorded. */
FMOE_API int fmoe_stage_timer_create(int32_t max_calls, void** timer);
FMOE_API int fmoe_stage_timer_destroy(void* timer);
/* Forget recorded calls (the events are reused). */
FMOE_API int fmoe_stage_timer_reset(void* timer);
/* Number of forward calls recorded since the last reset. */
FMOE_API int fmoe_stage_timer_calls(void* timer);
/* Waits for call `call` to finish on the device and writes its FMOE_STAGES stage durations in ms. */
FMOE_API int fmoe_stage_timer_read(void* timer, int32_t call, float* stage_ms);

/* ---- W8A8 routed-expert MoE ------------------------------------------------------------------ */

/* Workspace size and layout for fmoe_w8a8_forward (the reference keeps the same buffers in a
 * thread-local RuntimeScratch, csrc/moe/arm/i8mm_w8a8/kernels.cpp:118-182). */
FMOE_API int fmoe_w8a8_workspace_layout(int64_t tokens, int32_t top_k, int32_t experts, int32_t hidden, int32_t inter,
                               fmoe_workspace_layout* layout);

/* The W8A8 forward: route lists, per-route int8 activation quantisation, grouped gate_up GEMM with
 * dequant + clamp-10 SwiGLU + bf16 store, row requantisation, grouped down GEMM with dequant into
 * fp32 route rows, fixed-order top-k merge.  Replaces fused_moe_w8a8_tiled_async_plan_v2
 * (csrc/moe/arm/i8mm_w8a8/kernels.cpp:463-694).  `config` may be NULL (defaults). */
FMOE_API int fmoe_w8a8_forward(const void* x, const int8_t* w13, const float* s13, const int8_t* w2, const float* s2,
                      const float* topk_weights, const int64_t* topk_ids, int64_t tokens, int32_t top_k,
                      int32_t experts, int32_t hidden, int32_t inter, const fmoe_config* config, void* out,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Per-output-channel weight quantiser: scale = amax/127 (1 if the row is zero),
 * q = clamp(round_half_even(w/scale), +-127).  Replaces the quantiser inside
 * fused_moe_w8a8_tiled_prepare_weights (csrc/moe/arm/i8mm_w8a8/kernels.cpp:446-461).
 * w[rows, cols] bf16 -> q[rows, cols] int8, scale[rows] fp32. */
FMOE_API int fmoe_quantize_weight_rows(const void* w, int64_t rows, int32_t cols, int8_t* q, float* scale, void* stream);

/* Row quantiser stage hook: x[rows, cols] bf16 -> q int8 + scale fp32 with the chosen numerics
 * (quantize_bf16_row, csrc/moe/arm/i8mm_w8a8/kernels.cpp:211-228). */
FMOE_API int fmoe_quantize_rows(const void* x, int64_t rows, int32_t cols, int32_t numerics, int8_t* q, float* scale,
                       void* stream);

/* Route build without any allocation or caller workspace.  It has no counterpart in the reference, whose
 * route lists are std::vectors grown on the calling thread.  It exists for hosts that must not allocate
 * device memory while serving -- a server that gave all of HBM to its KV-cache pool, a runtime with a frozen
 * memory plan -- and so cannot provide the forward calls' workspace: the histograms and scan temporaries
 * live in a 528 KB array inside the library's device image (one per GPU that loads the library, held until
 * the process exits).  Limits: tokens * top_k <= 131072 and experts <= 512; larger requests are refused
 * with FMOE_ERR_INVALID_ARGUMENT.  The first call on each device looks the array's device address up
 * (cudaGetSymbolAddress); make that first call during start-up, before any stream capture.  Every call
 * uses the same array, so two calls that overlap on the GPU (different streams, or threads) race: issue
 * them on one stream.  Inputs and outputs are the caller's: counts[E], offsets[E+1], sorted_routes[T*K],
 * row_expert[T*K] as in fmoe_workspace_layout, status_out[2] = (error code, detail) as fmoe_read_status
 * would report them.  No cudaMalloc, cudaFree or other allocating call is made. */
FMOE_API int fmoe_route_build_noalloc(const int64_t* topk_ids, int64_t tokens, int32_t top_k, int32_t experts,
                                      int32_t* counts, int32_t* offsets, int32_t* sorted_routes, int32_t* row_expert,
                                      int32_t* status_out, void* stream);

/* ---- BF16 routed-expert MoE ------------------------------------------------------------------ */

FMOE_API int fmoe_bf16_workspace_layout(int64_t tokens, int32_t top_k, int32_t experts, int32_t hidden, int32_t inter,
                               fmoe_workspace_layout* layout);

/* The BF16 forward: route lists, row gather, grouped gate_up GEMM (fp32 accumulate) with
 * SiLU(gate)*up -> bf16, grouped down GEMM into fp32 route rows, tree/chain top-k merge.
 * Replaces fused_moe_bf16_tiled / fused_moe_bf16_tiled_async_plan_v2
 * (csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:6376, :9394). */
FMOE_API int fmoe_bf16_forward(const void* x, const void* w13, const void* w2, const float* topk_weights,
                      const int64_t* topk_ids, int64_t tokens, int32_t top_k, int32_t experts, int32_t hidden,
                      int32_t inter, const fmoe_config* config, void* out, void* workspace, size_t workspace_bytes,
                      void* stream);

/* ---- W8A16 routed-expert MoE ----------------------------------------------------------------- */

/* int8 weights with per-output-channel fp32 scales (layouts of the W8A8 entry point) and 16-bit activations:
 * value = (sum_k x[k] * q[n, k]) * scale[n] with the sum taken in one of the two forms of fmoe_config.w8a16_form
 * (16-bit fixed point per row on the int8 tensor cores, or bf16 activations against weights widened to bf16 with fp32
 * accumulation), then the BF16 path's activation, fp32 route rows and tree / chain merge.  Replaces fused_moe_w8a16_tiled_async_plan_v2
 * (csrc/moe/common/api.h:113-124; csrc/moe/arm/common/fused_moe_bf16_tiled.cpp:8740-8760) in its "scale the
 * accumulator" form; the reference's cache_dequant variant, which rounds q * scale to bf16 before multiplying, is
 * not reproduced (results agree to the BF16 tolerance).  Workspace: fmoe_bf16_workspace_layout.  No biases. */
FMOE_API int fmoe_w8a16_forward(const void* x, const int8_t* w13, const float* s13, const int8_t* w2, const float* s2,
                                const float* topk_weights, const int64_t* topk_ids, int64_t tokens, int32_t top_k,
                                int32_t experts, int32_t hidden, int32_t inter, const fmoe_config* config, void* out,
                                void* workspace, size_t workspace_bytes, void* stream);

/* ---- expert-parallel building blocks ------------------------------------------------------------
 *
 * The reference has no expert parallelism (it rejects expert id remapping,
 * csrc/moe/arm/i8mm_w8a8/kernels.cpp:488): these entry points have no counterpart there.  Ranks own
 * contiguous blocks of experts_global / world experts; tokens stay data-parallel.  The exchange itself
 * (two all-to-all-v) is the caller's: NCCL through torch.distributed in fused_cpp_b200/ep.py.  Every route
 * keeps the single-GPU arithmetic -- quantised where its token lives (quantize_bf16_row,
 * kernels.cpp:211-228), multiplied where its expert lives (run_stage + epilogues, :328-368, :230-257),
 * merged in slot order where its token lives (:675-688) -- so a sharded call returns the same bits. */

FMOE_API size_t fmoe_ep_dispatch_workspace_bytes(int64_t tokens, int32_t top_k, int32_t world);

/* Source side, before the exchange: sort this rank's T*K routes by destination rank (stable), and lay the
 * payload out in that order: send_rows[T*K, H] (int8 quantised per route when int8 != 0, else bf16 copies),
 * send_scale[T*K] (int8 only), send_expert[T*K] = expert id local to the destination, send_order[T*K] = the
 * flat route id t*K+slot of each send position, dest_counts[world] = routes per destination.
 * shared_rank >= 0: the id experts_global names a shared expert replicated on every rank (the reference's
 * synthetic expert E, src/fused_cpp/moe/bf16_tiled.py:1007-1013); those routes stay on shared_rank (the
 * caller's own rank) with local expert id experts_global / world.  shared_rank = -1: no shared expert. */
FMOE_API int fmoe_ep_dispatch_prepare(const void* x, const int64_t* topk_ids, int64_t tokens, int32_t top_k,
                                      int32_t experts_global, int32_t world, int32_t shared_rank, int32_t hidden, int32_t int8,
                                      int32_t numerics, int32_t* dest_counts, int32_t* send_order, void* send_rows,
                                      float* send_scale, int64_t* send_expert, void* workspace,
                                      size_t workspace_bytes, void* stream);

/* Expert side: the grouped gate_up / down GEMMs over received rows (one route per row, rows_expert = local
 * expert id); route_out[R, H] fp32 comes back in the order the rows were given.  Workspace as
 * fmoe_*_workspace_layout(tokens = R, top_k = 1, experts = local experts). */
FMOE_API int fmoe_w8a8_expert_rows_forward(const int8_t* rows_q, const float* rows_scale, const int64_t* rows_expert,
                                           int64_t rows, const int8_t* w13, const float* s13, const int8_t* w2,
                                           const float* s2, int32_t experts, int32_t hidden, int32_t inter,
                                           const fmoe_config* config, float* route_out, void* workspace,
                                           size_t workspace_bytes, void* stream);
FMOE_API int fmoe_bf16_expert_rows_forward(const void* rows, const int64_t* rows_expert, int64_t row_count,
                                           const void* w13, const void* w2, int32_t experts, int32_t hidden,
                                           int32_t inter, const fmoe_config* config, float* route_out,
                                           void* workspace, size_t workspace_bytes, void* stream);

/* Source side, after the exchange back: returned_rows[T*K, H] fp32 in send order are scattered to
 * route_out[flat route] (scratch of T*K*H floats) and merged with topk_weights into out[T, H] bf16;
 * tree_merge = 1 selects the BF16 path's pairwise order, 0 the W8A8 fused chain. */
FMOE_API int fmoe_ep_combine_finish(const float* returned_rows, const int32_t* send_order, const float* topk_weights,
                                    int64_t tokens, int32_t top_k, int32_t hidden, int32_t tree_merge,
                                    float* route_out, void* out, void* stream);

/* ---- dense W8A8 linear ----------------------------------------------------------------------- */

/* Workspace bytes for the dense calls below (quantised rows, scales, work items, status block, and for at most 16
 * rows the int32 table in which the K-split parts of a product meet; n = the widest N that will use the workspace.
 * A call given less than this for its N runs without the split). */
FMOE_API size_t fmoe_i8gemm_workspace_bytes(int64_t rows, int32_t k, int32_t n);

/* out[M,N] = dequant( quant_rows(x[M,K]) @ w^T ) (+ bias): per-row dynamic int8 quantisation
 * (scale = amax/127, 1 for a zero row; q = clamp(nearbyint(x/scale), -128, 127)), int32 accumulate on
 * the tensor cores, value = (acc * x_scale[m]) * w_scale[n] (+ bias[n]).  Replaces i8gemm_dynamic_scaled_mm
 * (csrc/i8gemm.cpp:318-452; scalar-fallback arithmetic :384-399, :147-165).
 * w is [N, Kp] int8 with Kp = K rounded up to 16 and the padding zero (what i8gemm_prepare's packed
 * weight is on this backend, csrc/i8gemm.cpp:280-316); w_scale[N] and bias[N] fp32, bias may be NULL;
 * x_is_bf16 / out_is_bf16 select bf16 (else fp32) element types. */
FMOE_API int fmoe_i8gemm_dynamic_scaled_mm(const void* x, int32_t x_is_bf16, int64_t rows, int32_t k, const int8_t* w,
                                           const float* w_scale, const float* bias, int32_t n, void* out,
                                           int32_t out_is_bf16, void* workspace, size_t workspace_bytes, void* stream);

/* Two bf16-output GEMMs over one shared activation quantisation (clamp +-127, no bias).  Replaces
 * i8gemm_dynamic_scaled_mm_pair (csrc/i8gemm.cpp:454-570; scalar arithmetic :492-506). */
FMOE_API int fmoe_i8gemm_dynamic_scaled_mm_pair(const void* x_bf16, int64_t rows, int32_t k, const int8_t* first_w,
                                                const float* first_scale, int32_t first_n, void* first_out,
                                                const int8_t* second_w, const float* second_scale, int32_t second_n,
                                                void* second_out, void* workspace, size_t workspace_bytes, void* stream);

/* ---- router front-end ------------------------------------------------------------------------- */

#define FMOE_SCORING_SOFTMAX 0
#define FMOE_SCORING_SIGMOID 1

/* The step in front of the path: expert scores -> top_k ids and routing weights, in the types the forward entry
 * points take, so that the ids go from the router to the route build without leaving the GPU.
 *   scoring softmax: p = softmax(logits[t, :]);  sigmoid: p = 1 / (1 + exp(-logits[t, :]))
 *   selection:       without a bias the top_k experts by logit (the same experts as by p, since both scorings are
 *                    monotone, and free of the rounding of exp); with selection_bias[e] the top_k by p + bias (the
 *                    bias only steers the choice); ties to the lower expert id
 *   weights:         p of the chosen experts, divided by their sum when renormalize != 0, times
 *                    routed_scaling_factor
 * The reference takes topk_weights / topk_ids as inputs (src/fused_cpp/moe/naive.py:4-7) and its callers compute
 * them in PyTorch; there is no reference kernel to match, parity is against torch.softmax / torch.topk on the
 * same logits (ids equal to torch.topk of the logits, weights to fp32 rounding).  experts <= 2048, top_k <= min(32, experts). */
FMOE_API int fmoe_router_topk(const float* logits, const float* selection_bias, int64_t tokens, int32_t experts, int32_t top_k,
                              int32_t scoring, int32_t renormalize, float routed_scaling_factor, float* topk_weights,
                              int64_t* topk_ids, void* stream);

/* ---- expert parallelism over peer memory --------------------------------------------------------- */

/* The same sharding as fmoe_ep_dispatch_prepare / fmoe_*_expert_rows_forward / fmoe_ep_combine_finish, with the row
 * exchanges and the synchronisation done by the kernels themselves instead of by a collective library: every
 * rank owns one "slab" (receive rows, their scale / local expert / return address, the fp32 result rows of its
 * own routes, row counts and barrier flags), exported by IPC handle and mapped by every other rank of the box.
 *     fmoe_ep_peer_dispatch   sorts this rank's routes by global expert id, tells every rank its counts per expert
 *                             (flag barrier with a payload), derives from the full count table where each of its
 *                             rows belongs in the owner's slab, then quantises each token once and stores its
 *                             rows straight to those final, expert-sorted positions; second flag barrier;
 *     fmoe_ep_peer_experts    the grouped GEMMs directly over the received rows (no route build, no gather); the
 *                             down GEMM's epilogue stores every result row straight into the slab of the rank
 *                             the route came from, tile by tile while the GEMM runs; third flag barrier;
 *     fmoe_ep_peer_combine    merges this rank's result rows.
 * Only plain stores cross NVLink; all loads (TMA included) read local memory.  Nothing synchronises with the host
 * and no collective library is involved after set-up.  The barrier waits are bounded (5 s, or
 * FUSED_CPP_MOE_EP_WAIT_MS): a rank that never arrives ends the wait with FMOE_ERR_DEVICE_WAIT in the status
 * block (fmoe_ep_peer_read_status), not with a hung GPU.  After a wait that gave up the rest of the forward sends
 * nothing and multiplies nothing (the row counts the later stages trust are cleared; return addresses are checked
 * before anything is stored through them); the output of that forward is undefined, the status says so.
 * Every rank must make the same sequence of calls.
 * Results are bit-identical to the single-GPU forward.  No counterpart in the reference, which rejects expert
 * parallelism (csrc/moe/arm/i8mm_w8a8/kernels.cpp:488). */
typedef struct fmoe_ep_peer_context fmoe_ep_peer_context;

/* Allocates the slab (sized for the worst case: every route of `world` ranks of tokens_max tokens lands here)
 * and the local scratch.  top_k counts the shared-expert route if there is one; local_experts likewise.
 * return_bf16 != 0 (opt-in): the result rows travel back as bf16 instead of fp32, which halves the return
 * traffic; the merge then starts from rounded rows, so the output is no longer bit-identical to the single-GPU
 * forward: relative L2 stays below 5e-3, single elements move by a bf16 step. */
FMOE_API int fmoe_ep_peer_create(int32_t world, int32_t rank, int64_t tokens_max, int32_t top_k, int32_t hidden, int32_t inter,
                                 int32_t local_experts, int32_t int8, int32_t return_bf16, fmoe_ep_peer_context** context);
/* 64-byte IPC handle of this rank's slab, to be given to every other rank. */
FMOE_API int fmoe_ep_peer_handle(fmoe_ep_peer_context* context, void* handle64);
/* handles: world x 64 bytes, entry r = rank r's handle (this rank's own entry is ignored). */
FMOE_API int fmoe_ep_peer_connect(fmoe_ep_peer_context* context, const void* handles);
/* The same connection for ranks that can already address one another's slabs: several contexts inside one process
 * (one per GPU with peer access enabled, or, for tests, several on one GPU).  slabs[r] = fmoe_ep_peer_slab_address
 * of rank r's context as valid in this process (this rank's own entry is ignored).  No IPC handle is opened. */
FMOE_API void* fmoe_ep_peer_slab_address(fmoe_ep_peer_context* context);
FMOE_API int fmoe_ep_peer_connect_addresses(fmoe_ep_peer_context* context, const void* const* slabs);
FMOE_API void fmoe_ep_peer_destroy(fmoe_ep_peer_context* context);
FMOE_API int64_t fmoe_ep_peer_slab_bytes(const fmoe_ep_peer_context* context);
/* shared_rank >= 0: expert id experts_global is the replicated shared expert, served by the calling rank itself
 * (pass the own rank; -1 = no shared expert).  Contains the first two barriers. */
FMOE_API int fmoe_ep_peer_dispatch(fmoe_ep_peer_context* context, const void* x_bf16, const int64_t* topk_ids, int64_t tokens,
                                   int32_t experts_global, int32_t shared_rank, int32_t numerics, void* stream);
/* Grouped GEMMs over the received rows; result rows go to the source ranks' slabs.  Ends with the third barrier. */
FMOE_API int fmoe_ep_peer_experts(fmoe_ep_peer_context* context, const void* w13, const float* s13, const void* w2, const float* s2,
                                  const fmoe_config* config, void* stream);
/* Merge of this rank's result rows in the reference's slot order (tree_merge: the BF16 path's pairwise tree). */
FMOE_API int fmoe_ep_peer_combine(fmoe_ep_peer_context* context, const float* topk_weights, int64_t tokens, int32_t tree_merge,
                                  void* out_bf16, void* stream);
/* First device-side error of the last dispatch and expert stage (synchronises the stream). */
FMOE_API int fmoe_ep_peer_read_status(fmoe_ep_peer_context* context, void* stream, int32_t* dispatch_error, int32_t* expert_error);

#ifdef __cplusplus
}
#endif

#endif /* FUSED_MOE_B200_H_ */
