// Launchers of the individual kernels; the C ABI in api.cu sequences them.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace fmoe {

constexpr int kUnitRoutes = 512;   // routes per warp in the route-build kernels
constexpr int kMaxExperts = 2048;  // bound of the per-warp shared-memory histograms

// ---- api.cu
int report_error(int code, const char* text);

// ---- route.cu
size_t route_scratch_bytes(int64_t routes, int experts);
// The work-item lists a route build fills: a and b for the gate_up and the down GEMM (tile heights tile_a,
// tile_b).  With split_rows > 0, a and b hold only the experts with at most split_rows rows and c and d
// (tile big_tile) the experts with more; every list has room for max_items items of four ints.
struct ItemLists {
  int tile_a, tile_b;
  int* items_a;
  int* items_b;
  int max_items;
  int split_rows;
  int big_tile;
  int* items_c;
  int* items_d;
};
inline ItemLists no_item_lists() { return ItemLists{16, 16, nullptr, nullptr, 0, 0, 0, nullptr, nullptr}; }
cudaError_t launch_route_build(const int64_t* topk_ids, int64_t routes, int experts, const ItemLists& lists, int* status, int* counts,
                               int* offsets, int* sorted_routes, int* row_expert, int* scratch, cudaStream_t stream,
                               int* route_pos = nullptr);

// Work items from per-expert counts / offsets of rows that are already in expert order (scratch: 2 * experts + 1 ints).
cudaError_t launch_items_from_counts(int experts, const int* counts, const int* offsets, const ItemLists& lists, int* scratch, int* status,
                                     cudaStream_t stream);

// ---- quant.cu
// Quantise rows of a bf16 matrix to int8 with one fp32 scale per row.  When `sorted_routes` is
// non-null, output row p reads source row sorted_routes[p] / top_k (gather by token).
// weight_mode: scale of an all-zero row is 1 and rounding is ties-to-even with division (weight prep).
// valid_rows (nullable, device): rows at or beyond *valid_rows are skipped (routes dropped for a bad id).
cudaError_t launch_quantize_rows(const uint16_t* x, int64_t out_rows, int cols, const int* sorted_routes, int top_k,
                                 const int* valid_rows, int numerics, int weight_mode, int8_t* q, float* scale,
                                 cudaStream_t stream);
// Quantise every token row once and write it to the sorted positions of its top_k routes
// (route_pos[t*top_k+slot], -1 = dropped): same bits as quantising per route, one read of x per token.
cudaError_t launch_quantize_tokens_scatter(const uint16_t* x, int64_t tokens, int cols, int top_k, const int* route_pos,
                                           int numerics, int8_t* q, float* scale, cudaStream_t stream);
// W8A16 in its fixed-point form: bf16 row p (gathered by token when sorted_routes is given) -> 16-bit fixed point per
// row, stored as two int8 rows (high plane at 2p, low plane at 2p + 1 of `planes`), row scale in scale[p].
cudaError_t launch_split_rows_planes(const uint16_t* x, int64_t out_rows, int cols, const int* sorted_routes, int top_k,
                                     const int* valid_rows, int8_t* planes, float* scale, cudaStream_t stream);
// The same split once per token, written to the sorted positions of its top_k routes (route_pos[t * top_k + slot],
// -1 = dropped).
cudaError_t launch_split_tokens_scatter_planes(const uint16_t* x, int64_t tokens, int cols, int top_k, const int* route_pos, int8_t* planes,
                                               float* scale, cudaStream_t stream);
// Same for fp32 sources (dense linear).  clamp_low is -128 or -127.
cudaError_t launch_quantize_rows_dense(const void* x, int x_is_bf16, int64_t rows, int cols, int cols_padded, int clamp_low,
                                       int8_t* q, float* scale, int row_tile, int max_items, int* items, int* status,
                                       cudaStream_t stream);
// Copy bf16 rows into expert-sorted order: out[p] = x[sorted_routes[p] / top_k].
cudaError_t launch_gather_rows(const uint16_t* x, int64_t out_rows, int cols, const int* sorted_routes, int top_k,
                               const int* valid_rows, uint16_t* out, cudaStream_t stream);

// out[i] = in[index[i]] for fp32 scalars (activation scales following their rows).
cudaError_t launch_gather_scalars(const float* in, int64_t n, const int* index, const int* valid_rows, float* out,
                                  cudaStream_t stream);

// ---- ep.cu: helpers of the expert-parallel dispatch / combine
// dest[i] = ids[i] / experts_per_rank as int64 (ids outside [0, experts_global) become -1).  With
// shared_rank >= 0 the id experts_global (the replicated shared expert) maps to shared_rank.
cudaError_t launch_dest_ranks(const int64_t* ids, int64_t n, int experts_global, int experts_per_rank, int shared_rank,
                              int64_t* dest, cudaStream_t stream);
// local[p] = ids[order[p]] % experts_per_rank (experts_per_rank for the shared expert) for the first *valid_rows positions.
cudaError_t launch_local_experts(const int64_t* ids, const int* order, int64_t n, const int* valid_rows, int experts_global,
                                 int experts_per_rank, int64_t* local, cudaStream_t stream);
// route_out[order[p], :] = rows[p, :] (fp32 rows of `hidden` columns).
cudaError_t launch_scatter_rows_f32(const float* rows, const int* order, int64_t n, const int* valid_rows, int hidden,
                                    float* route_out, cudaStream_t stream);

// Peer-memory path.  Every rank owns one slab with the same layout (byte offsets below); peer_slabs[r] is the
// address of rank r's slab as mapped into this process.
struct PeerSlabLayout {
  size_t rows;       // [capacity, H] int8 or bf16: received rows in expert order (sources in rank order inside an expert)
  size_t scale;      // [capacity] fp32: activation scale of each received row (int8)
  size_t source;     // [capacity] int2: (source rank, flat route id at the source)
  size_t route_out;  // [local routes, H] fp32 (or bf16): result rows of this rank's own routes, written by the expert ranks
  size_t counts;     // [world, row stride] int: route counts per global expert of every source rank
  size_t flags;      // [world] uint32: barrier epochs, one per source rank
  size_t total;
};
// zero_on_fail (nullable): zero_ints ints that are cleared when the wait gives up (row counts the next stages trust).
cudaError_t launch_peer_barrier(const uint64_t* peer_slabs, const PeerSlabLayout& slab, const int* payload, int payload_ints, int world,
                                int rank, unsigned* epoch_counter, int* status, unsigned long long limit_ns, cudaStream_t stream,
                                int* zero_on_fail = nullptr, int zero_ints = 0);
// status: the dispatch status block; after a failed count exchange the layout publishes empty lists.
cudaError_t launch_peer_layout(const int* count_matrix, int world, int rank, int experts_global, int per_rank, int has_shared,
                               int row_stride, int* send_base, int* local_counts, int* local_offsets, const int* status,
                               cudaStream_t stream);
cudaError_t launch_peer_dispatch(bool int8, const uint16_t* x, const int64_t* topk_ids, int64_t tokens, int cols, int top_k,
                                 const int* route_pos, const int* expert_offsets, const int* send_base, const PeerSlabLayout& slab,
                                 const uint64_t* peer_slabs, int rank, int experts_global, int experts_per_rank, int has_shared,
                                 int numerics, int64_t capacity, int* status, cudaStream_t stream);
// Return addresses outside [0, world) x [0, routes_max) are reported in `status` and replaced by scrap_row (local).
cudaError_t launch_peer_row_ptrs(const int* valid_rows, int64_t capacity, const void* source, const uint64_t* peer_slabs,
                                 size_t route_out_offset, int row_bytes, uint64_t* row_out_ptrs, int world, int64_t routes_max,
                                 void* scrap_row, int* status, cudaStream_t stream);

// ---- router.cu: scores -> top-k ids and routing weights, one warp per token (experts <= 2048, top_k <= 32)
cudaError_t launch_router_topk(const float* logits, const float* selection_bias, int64_t tokens, int experts, int top_k, int sigmoid,
                               int renormalize, float scaling, float* topk_weights, int64_t* topk_ids, cudaStream_t stream);

// ---- merge.cu
// W8A8: out[t] = bf16( fma chain over slots of route_out[t*K+slot] * w[t,slot] ).
// BF16: pairwise tree for K in {2,4,6,8}, chain otherwise.
// route_pos (nullable): sorted position of every flat route, -1 = dropped by the route build; such rows count as zeros.
cudaError_t launch_merge(const float* route_out, const float* topk_weights, int64_t tokens, int top_k, int hidden,
                         int tree, uint16_t* out, cudaStream_t stream, const int* route_pos = nullptr);
// Same with the route rows stored as bf16 (opt-in compact return of the expert-parallel path).
cudaError_t launch_merge_bf16_rows(const uint16_t* route_out, const float* topk_weights, int64_t tokens, int top_k, int hidden,
                                   int tree, uint16_t* out, cudaStream_t stream, const int* route_pos = nullptr);

// ---- grouped GEMM, shared argument block
struct GroupedGemmArgs {
  const void* a_rows;        // [rows, K] int8 or bf16, expert-sorted
  const void* weights;       // [E, N_total, K] int8 or bf16
  const float* a_scale;      // [rows] (int8) or null
  const float* w_scale;      // [E, N_total] (int8) or null
  const int* items;          // (expert, first row, rows, 0) per work item
  const int* status;         // status block: item counts are read from it
  int item_count_word;       // kStatusItems or kStatusItemsB
  int max_items;
  const int* sorted_routes;  // down GEMM: flat route id of each sorted row
  int experts;
  int k;                     // reduction length (H for gate_up, I for down)
  int n_out;                 // output channels per row: I (gate_up, gate/up pairs) or H (down)
  int numerics;
  float swiglu_limit;
  uint16_t* y;               // gate_up output bf16 [rows, I]
  float* route_out;          // down output fp32 [T*K, H], row = flat route id
  void* dump_acc;            // optional raw accumulators [rows, N_total], sorted-row order
  int64_t total_rows;
  int row_tile;              // rows per work item
  int* status_rw;            // writable status block (device-side error reports)
  // Dense-linear mode of the down epilogue: out[row, n] = dequant (+ bias[n]) as fp32 or bf16, no scatter.
  void* dense_out;
  int dense_out_bf16;
  const float* bias;
  // Down GEMM, optional: byte address of the fp32 output row of every sorted row.  Overrides route_out +
  // sorted_routes; the rows may lie in another GPU's memory (expert-parallel return path, plain stores).
  const uint64_t* row_out_ptrs;
  // BF16 path only: per-expert bias added to the fp32 accumulators before the activation (gate_up: [E, 2I], gate
  // channels then up channels) or before the store (down: [E, H]); null = none.  `activation` selects the gated
  // activation of the gate_up epilogue: FMOE_ACT_SILU (with swiglu_limit), FMOE_ACT_GELU, FMOE_ACT_SWIGLUOAI.
  const float* expert_bias;
  int activation;
  int w8a16;                 // int8 weights with w_scale and 16-bit activations: 1 = bf16 rows, the one-SM kernel widens the weight
                             // tile to bf16; 2 = two int8 planes per route (a_rows holds 2 * total_rows rows, a_scale one
                             // scale per route, row_tile counts plane rows), the int8 one-SM kernel pairs accumulator columns
  int gate_up_one_box;       // two-SM gate_up: the weight rows of a stage arrive as one 16 KB TMA box (set by the launcher)
  // Dense GEMM over few rows (one-SM kernel): the K range of every (row tile, channel block) is cut into dense_splits
  // parts that run as work units of their own, so that a product with few channel blocks still fills the SMs.  The
  // parts add their int32 accumulators into dense_partial[rows, n_out] (zero on entry) and count themselves in
  // dense_counters[unit] (zero on entry); the part that arrives last dequantises and stores.  0 or 1 = no split.
  int dense_splits;
  int* dense_partial;
  int* dense_counters;
  int route_out_bf16;        // the result rows are stored as bf16 (2 bytes per channel, rows 2 * n_out bytes apart) instead of fp32
  // Diagnostic build only (compiled with -DFMOE_DIAG, the separate libfused_moe_b200_diag.so; the product library
  // ignores the field): bit 0 = epilogue does no work, bit 1 = producer loads nothing, bit 2 = no MMA is issued.
  int diag;
};

// The stage switches above exist only in the diagnostic build; in the product build the tests fold to `false`.
#ifdef FMOE_DIAG
#define FMOE_DIAG_BIT(args, bit) (((args).diag & (bit)) != 0)
#else
#define FMOE_DIAG_BIT(args, bit) false
#endif

// Launch set-up that belongs to a device, not to the process: the opt-in to more than 48 KB of dynamic shared
// memory (a function attribute) and the SM count are remembered per device ordinal.
constexpr int kMaxDevices = 64;
inline int current_device_ordinal() {
  int device = 0;
  cudaGetDevice(&device);
  return device;
}
struct PerDeviceOnce {
  bool done[kMaxDevices] = {};
  // True when `device` still needs its set-up (ordinals beyond the table are set up on every call).
  bool needed(int device) const { return device < 0 || device >= kMaxDevices || !done[device]; }
  void mark(int device) {
    if (device >= 0 && device < kMaxDevices) done[device] = true;
  }
};
inline int sm_count_of_current_device() {
  static int counts[kMaxDevices] = {};
  const int device = current_device_ordinal();
  if (device >= 0 && device < kMaxDevices && counts[device] > 0) return counts[device];
  int count = 0;
  cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
  if (count <= 0) count = 148;
  if (device >= 0 && device < kMaxDevices) counts[device] = count;
  return count;
}

// ---- simt_gemm.cu: CUDA-core grouped GEMM of the diagnostic library only (work items of at most 8 rows)
constexpr int kSimtRowTile = 8;
cudaError_t launch_simt_grouped_gemm(const GroupedGemmArgs& args, bool int8, bool gate_up, cudaStream_t stream);

// ---- umma_gemm.cu: tcgen05 grouped GEMM
bool umma_row_tile_supported(int row_tile);
cudaError_t launch_umma_grouped_gemm(const GroupedGemmArgs& args, bool int8, bool gate_up, cudaStream_t stream);

// ---- umma2_gemm.cu: two-SM (cta_group::2) grouped GEMM, 256-row work items.  Selected by row tile 512.
constexpr int kPairRowTile = 512;
bool umma_pair_supported(bool gate_up, int n_out, int64_t output_rows);  // else callers use the one-SM kernel on the same items
cudaError_t launch_umma_pair_grouped_gemm(const GroupedGemmArgs& args, bool int8, bool gate_up, cudaStream_t stream);

// ---- probe.cu (diagnostic library only): tcgen05.mma issue-rate probe (128 x n x 32-byte MMAs back to back on every CTA)
cudaError_t launch_mma_rate_probe(bool int8, int n, int iterations, int mode, int blocks, int* status, cudaStream_t stream);
// The same for two-SM MMAs (256 x n x 32 bytes issued by the leader of every two-CTA cluster).
cudaError_t launch_mma_rate_pair_probe(bool int8, int n, int iterations, int mode, int blocks, int* status, cudaStream_t stream);

}  // namespace fmoe
