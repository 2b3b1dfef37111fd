// C ABI of the library: argument validation, workspace layout and the kernel sequence of each
// forward call.  See include/fused_moe_b200.h for the contract of every entry point.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#ifdef FMOE_DIAG
#include "diag.h"
#endif

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* format, ...) {
  va_list list;
  va_start(list, format);
  vsnprintf(g_error, sizeof(g_error), format, list);
  va_end(list);
  return code;
}

int cuda_fail(cudaError_t error, const char* what) {
  return fail(FMOE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(error));
}

size_t align_up(size_t value, size_t quantum) { return (value + quantum - 1) / quantum * quantum; }

int check_device() {
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return cuda_fail(error, "cudaGetDevice");
  static thread_local int checked_device = -1;
  if (checked_device == device) return FMOE_OK;
  if (!fmoe_device_supported(device)) {
    return fail(FMOE_ERR_UNSUPPORTED_DEVICE, "device %d is not a compute capability 10.x GPU; this library has no other path", device);
  }
  checked_device = device;
  return FMOE_OK;
}

constexpr int kSplitRows = 64;  // experts with more rows than this go to the two-SM kernel when the tiles are automatic

int64_t max_items_for(int64_t routes, int experts) {
  // Upper bound on (expert, row tile) items for any tile height >= 8.
  return experts + routes / 8 + 1;
}

int check_shape(int64_t tokens, int top_k, int experts, int hidden, int inter) {
  if (tokens < 0 || top_k <= 0 || top_k > 32 || experts <= 0 || experts > fmoe::kMaxExperts) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "invalid shape: tokens=%lld top_k=%d (1..32) experts=%d (1..%d)",
                static_cast<long long>(tokens), top_k, experts, fmoe::kMaxExperts);
  }
  if (hidden <= 0 || inter <= 0 || hidden % 16 != 0 || inter % 16 != 0) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "H and I must be positive multiples of 16 (H=%d, I=%d)", hidden, inter);
  }
  if (tokens * top_k > (1ll << 30)) return fail(FMOE_ERR_INVALID_ARGUMENT, "too many routes");
  return FMOE_OK;
}

// with_route_out = false (peer-memory expert stage): the fp32 route rows live elsewhere and the region only
// holds one 8-byte output address per row; the sorted copy of the activation rows is not needed either.
int make_layout(bool int8, int64_t tokens, int top_k, int experts, int hidden, int inter, fmoe_workspace_layout* layout,
                bool with_route_out = true) {
  const int status = check_shape(tokens, top_k, experts, hidden, inter);
  if (status != FMOE_OK) return status;
  if (layout == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "layout is null");
  const size_t routes = static_cast<size_t>(tokens) * top_k;
  const size_t rows = routes > 0 ? routes : 1;
  const size_t max_items = static_cast<size_t>(max_items_for(routes, experts));
  size_t offset = 0;
  auto take = [&offset](size_t bytes) {
    const size_t begin = offset;
    offset = align_up(offset + bytes, 256);
    return begin;
  };
  memset(layout, 0, sizeof(*layout));
  layout->status = take(sizeof(int) * fmoe::kStatusWords);
  layout->counts = take(sizeof(int) * experts);
  layout->offsets = take(sizeof(int) * (experts + 1));
  layout->sorted_routes = take(sizeof(int) * rows);
  layout->row_expert = take(sizeof(int) * rows);
  layout->items = take(sizeof(int) * 4 * max_items * 4);  // four work-item lists (see fmoe::ItemLists)
  layout->scratch = take(fmoe::route_scratch_bytes(routes, experts));
  layout->a_rows = take(with_route_out ? rows * hidden * (int8 ? 1 : 2) : 256);
  layout->a_scale = take(sizeof(float) * rows);
  layout->y = take(rows * inter * 2);
  // W8A16 (which uses the 16-bit layout) holds the two int8 planes of the intermediate in a_rows when they fit
  // there (inter <= hidden: the activation planes are dead by then), else here.
  layout->yq = take(int8 ? rows * inter : (inter > hidden ? rows * inter * 2 : 0));
  layout->y_scale = take(sizeof(float) * rows);
  layout->route_out = take(with_route_out ? sizeof(float) * rows * hidden : sizeof(uint64_t) * rows);
  layout->route_pos = take(sizeof(int) * rows);
  layout->total_bytes = offset;
  return FMOE_OK;
}

// Row tile when the caller leaves it to the library and the batch has at most 64 tokens: an expert can then hold at
// most `tokens` rows, so the smallest tile that holds them all puts every expert in one work item whatever the
// routing looks like (the MMA's N follows the rows an item really has, a taller tile only costs shared memory:
// +0.4 % on uniformly routed decode, -26 % on Zipf-routed decode at T = 64).
int pick_row_tile(int requested, int64_t tokens, bool umma) {
  if (!umma) return fmoe::kSimtRowTile;
  if (requested != 0) return requested;
  if (tokens <= 16) return 16;
  if (tokens <= 32) return 32;
  return 64;
}

struct StageTimer {
  int max_calls = 0;
  int calls = 0;
  std::vector<cudaEvent_t> events;  // (FMOE_STAGES + 1) per call
};

struct Forward {
  bool int8;
  const void* x;
  const void* w13;
  const float* s13;
  const void* w2;
  const float* s2;
  const float* topk_weights;
  const int64_t* topk_ids;
  int64_t tokens;
  int top_k, experts, hidden, inter;
  // Expert-rows mode (expert-parallel receive side): `x` holds rows that are already quantised (int8, with
  // rows_scale) or gathered (bf16), one route per row, topk_ids[R,1] = the row's local expert; the merge is
  // skipped and the fp32 route rows go to route_out_override in the order the rows were given.
  const float* rows_scale = nullptr;
  float* route_out_override = nullptr;
  bool rows_mode = false;
  // Peer-memory expert stage: the rows already lie in expert order (sorted_counts[e] rows of local expert e from
  // sorted_offsets[e]; sorted_offsets[experts] = rows in all; both on the device) in a list of capacity `tokens`;
  // rows_source[row] = (source rank, flat route) and every result row is stored into the source rank's slab at
  // peer_slabs[rank] + peer_route_out_offset.  No route build and no gather happen here.
  const int* sorted_counts = nullptr;
  const int* sorted_offsets = nullptr;
  const void* rows_source = nullptr;
  const uint64_t* peer_slabs = nullptr;
  size_t peer_route_out_offset = 0;
  // W8A16: int8 weights with per-output-channel scales s13 / s2, bf16 activations (int8 = false: no activation
  // quantisation, the BF16 workspace and merge).
  bool w8a16 = false;
  bool peer_rows_bf16 = false;  // result rows travel as bf16 (opt-in, not bit-identical to the fp32 merge input)
  // Bounds of a valid return address (source rank < peer_world, flat route < peer_routes_max) and the local row
  // that takes the stores of a row whose return address is not valid.
  int peer_world = 0;
  int64_t peer_routes_max = 0;
  void* peer_scrap_row = nullptr;
};

int run_forward(const Forward& f, const fmoe_config* config, void* out, void* workspace, size_t workspace_bytes, void* stream_ptr) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  fmoe_workspace_layout layout;
  const bool peer = f.peer_slabs != nullptr;
  status = make_layout(f.int8, f.tokens, f.top_k, f.experts, f.hidden, f.inter, &layout, !peer);
  if (status != FMOE_OK) return status;
  if (f.tokens == 0) return FMOE_OK;
  if (f.x == nullptr || f.w13 == nullptr || f.w2 == nullptr || (f.topk_ids == nullptr && !peer)) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "null tensor pointer");
  }
  if (!f.rows_mode && (f.topk_weights == nullptr || out == nullptr)) return fail(FMOE_ERR_INVALID_ARGUMENT, "null tensor pointer");
  if (peer && (!f.rows_mode || f.sorted_counts == nullptr || f.sorted_offsets == nullptr || f.rows_source == nullptr ||
               f.peer_scrap_row == nullptr || f.peer_world <= 0)) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "peer-memory mode needs expert-sorted rows with device-side counts and their sources");
  }
#ifdef FMOE_DIAG
  if (peer && config != nullptr && config->gemm_impl == FMOE_GEMM_SIMT) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "peer-memory mode runs on the tensor-core GEMMs only");
  }
#endif
  if (f.rows_mode && ((f.route_out_override == nullptr && !peer) || (f.int8 && f.rows_scale == nullptr) || f.top_k != 1)) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "expert-rows mode needs route_out, row scales (int8) and one route per row");
  }
  if ((f.int8 || f.w8a16) && (f.s13 == nullptr || f.s2 == nullptr)) return fail(FMOE_ERR_INVALID_ARGUMENT, "null scale pointer");
  if (workspace == nullptr || workspace_bytes < layout.total_bytes) {
    return fail(FMOE_ERR_WORKSPACE, "workspace too small: %zu bytes given, %zu needed", workspace_bytes, layout.total_bytes);
  }
  if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail(FMOE_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  const uintptr_t align_mask = reinterpret_cast<uintptr_t>(f.x) | reinterpret_cast<uintptr_t>(f.w13) |
                               reinterpret_cast<uintptr_t>(f.w2) | reinterpret_cast<uintptr_t>(out) |
                               reinterpret_cast<uintptr_t>(f.route_out_override);
  if (align_mask % 16 != 0) return fail(FMOE_ERR_INVALID_ARGUMENT, "x, w13, w2, out and route_out must be 16-byte aligned");

  fmoe_config defaults;
  memset(&defaults, 0, sizeof(defaults));
  defaults.swiglu_limit = f.int8 ? 10.0f : 0.0f;
  const fmoe_config cfg = config ? *config : defaults;
  if (f.int8 && cfg.swiglu_limit != 10.0f) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "W8A8 supports only clamped SwiGLU limit 10.0");
  }
  if (!f.int8 && cfg.swiglu_limit != 0.0f && cfg.swiglu_limit != 10.0f) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "BF16 supports swiglu_limit 0 (plain SiLU) or 10.0");
  }
  if (cfg.route_rows_bf16 != 0 && cfg.route_rows_bf16 != 1) return fail(FMOE_ERR_INVALID_ARGUMENT, "route_rows_bf16 must be 0 or 1");
  if (cfg.activation != FMOE_ACTIVATION_SILU && cfg.activation != FMOE_ACTIVATION_GELU && cfg.activation != FMOE_ACTIVATION_SWIGLUOAI) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "unknown activation %d", cfg.activation);
  }
  if (f.int8 && (cfg.activation != FMOE_ACTIVATION_SILU || cfg.w13_bias != nullptr || cfg.w2_bias != nullptr)) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "W8A8 supports only the clamped SiLU activation and no w13_bias / w2_bias");
  }
  if (f.w8a16 && (cfg.w13_bias != nullptr || cfg.w2_bias != nullptr)) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "W8A16 takes no w13_bias / w2_bias");
  }
  if (cfg.w8a16_form != FMOE_W8A16_FIXED_POINT && cfg.w8a16_form != FMOE_W8A16_BF16_ACTIVATIONS) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "unknown w8a16_form %d", cfg.w8a16_form);
  }
  if (cfg.activation != FMOE_ACTIVATION_SILU && cfg.swiglu_limit != 0.0f) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "swiglu_limit is only valid with the SiLU activation");
  }
  if (cfg.numerics != FMOE_NUMERICS_TORCHREF && cfg.numerics != FMOE_NUMERICS_NATIVE) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "unknown numerics %d", cfg.numerics);
  }
#ifdef FMOE_DIAG
  if (cfg.gemm_impl < FMOE_GEMM_AUTO || cfg.gemm_impl > FMOE_GEMM_UMMA) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "unknown gemm_impl %d", cfg.gemm_impl);
  }
  const bool umma = cfg.gemm_impl != FMOE_GEMM_SIMT;
#else
  if (cfg.gemm_impl != FMOE_GEMM_AUTO && cfg.gemm_impl != FMOE_GEMM_UMMA) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "unknown gemm_impl %d (this library has one grouped-GEMM implementation, tcgen05)", cfg.gemm_impl);
  }
  const bool umma = true;
#endif
  const int64_t routes = f.tokens * f.top_k;
  // Above 64 tokens an expert can hold anything from one row to all of them, and the host does not know the routing.
  // Unless the caller fixed the tiles, the experts are then split on the device: those with at most 64 rows
  // go through the one-SM kernel (64-row tile, every weight byte streamed once), the others through the
  // two-SM kernel (256-row work items).  Up to 64 tokens no expert can exceed 64 rows and the tile follows
  // the batch size (pick_row_tile).
  // W8A16.  Its fixed-point form runs on the int8 kernels with two token rows (planes) per route: the kernel's row
  // tile is twice the routes of a work item, so an item holds at most 128 routes; above 64 tokens the experts are
  // split like W8A8's (thin ones to the one-SM kernel, the others to the two-SM kernel in 128-route items).  Its
  // bf16-activation form runs every expert through the one-SM kernel (the int8 -> bf16 widening lives there): no
  // split, and a 128-row tile above 64 tokens.
  const bool planes = f.w8a16 && umma && cfg.w8a16_form == FMOE_W8A16_FIXED_POINT;
  const bool split = umma && (!f.w8a16 || planes) && cfg.gate_up_tile == 0 && cfg.down_tile == 0 && f.tokens > kSplitRows;
  const bool w8a16_wide = f.w8a16 && !planes && f.tokens > kSplitRows;
  int tile_gu = split ? kSplitRows : (w8a16_wide && cfg.gate_up_tile == 0) ? 128 : pick_row_tile(cfg.gate_up_tile, f.tokens, umma);
  int tile_dn = split ? kSplitRows : (w8a16_wide && cfg.down_tile == 0) ? 128 : pick_row_tile(cfg.down_tile, f.tokens, umma);
  if (planes) {
    // Tiles given by the caller: 16..128 routes per item on the one-SM kernel, 512 = the two-SM kernel; 256 is cut to 128.
    if (tile_gu == 256) tile_gu = 128;
    if (tile_dn == 256) tile_dn = 128;
  } else if (f.w8a16) {
    // The token-major widening kernel holds a work item in the 128 lanes of one accumulator: taller tiles are cut to 128.
    tile_gu = tile_gu > 128 ? 128 : tile_gu;
    tile_dn = tile_dn > 128 ? 128 : tile_dn;
  }
  if (umma && (!fmoe::umma_row_tile_supported(tile_gu) || !fmoe::umma_row_tile_supported(tile_dn))) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "row tiles must be 16, 32, 64, 128, 256 or 512 = two-SM pairs (got %d, %d)", tile_gu, tile_dn);
  }
  // Tile 512 selects the two-SM kernel, whose work items hold up to 256 rows.
  const int pair_item_rows = planes ? 128 : 256;  // routes of a two-SM work item (256 token rows either way)
  const int item_rows_gu = tile_gu == fmoe::kPairRowTile ? pair_item_rows : tile_gu;
  const int item_rows_dn = tile_dn == fmoe::kPairRowTile ? pair_item_rows : tile_dn;

  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  char* base = static_cast<char*>(workspace);
  int* status_block = reinterpret_cast<int*>(base + layout.status);
  int* counts = reinterpret_cast<int*>(base + layout.counts);
  int* offsets = reinterpret_cast<int*>(base + layout.offsets);
  int* sorted_routes = reinterpret_cast<int*>(base + layout.sorted_routes);
  int* row_expert = reinterpret_cast<int*>(base + layout.row_expert);
  const int max_items = static_cast<int>(max_items_for(routes, f.experts));
  int* items_gu = reinterpret_cast<int*>(base + layout.items);
  int* items_dn = items_gu + 4 * static_cast<size_t>(max_items);
  int* items_gu_big = items_dn + 4 * static_cast<size_t>(max_items);
  int* items_dn_big = items_gu_big + 4 * static_cast<size_t>(max_items);
  const fmoe::ItemLists lists{item_rows_gu, item_rows_dn, items_gu, items_dn, max_items, split ? kSplitRows : 0, split ? pair_item_rows : 0,
                              items_gu_big, items_dn_big};
  int* scratch = reinterpret_cast<int*>(base + layout.scratch);
  float* a_scale = reinterpret_cast<float*>(base + layout.a_scale);
  uint16_t* y = reinterpret_cast<uint16_t*>(base + layout.y);
  float* y_scale = reinterpret_cast<float*>(base + layout.y_scale);
  float* route_out = f.rows_mode ? f.route_out_override : reinterpret_cast<float*>(base + layout.route_out);

  StageTimer* timer = static_cast<StageTimer*>(cfg.stage_timer);
  cudaEvent_t* marks = nullptr;
  if (timer != nullptr && timer->calls < timer->max_calls) {
    marks = timer->events.data() + static_cast<size_t>(timer->calls) * (FMOE_STAGES + 1);
    timer->calls += 1;
  }
  auto mark = [&](int index) {
    if (marks != nullptr) cudaEventRecord(marks[index], stream);
  };
  mark(0);
  cudaError_t error = cudaMemsetAsync(status_block, 0, sizeof(int) * fmoe::kStatusWords, stream);
  if (error != cudaSuccess) return cuda_fail(error, "cudaMemsetAsync(status)");
  uint64_t* row_out_ptrs = nullptr;
  if (peer) {
    // The rows arrived in expert order: only the work items and the output addresses remain to be made.
    error = fmoe::launch_items_from_counts(f.experts, f.sorted_counts, f.sorted_offsets, lists, scratch, status_block, stream);
    if (error != cudaSuccess) return cuda_fail(error, "work items");
    row_out_ptrs = reinterpret_cast<uint64_t*>(base + layout.route_out);
    error = fmoe::launch_peer_row_ptrs(f.sorted_offsets + f.experts, routes, f.rows_source, f.peer_slabs, f.peer_route_out_offset,
                                       f.hidden * (f.peer_rows_bf16 ? 2 : 4), row_out_ptrs, f.peer_world, f.peer_routes_max,
                                       f.peer_scrap_row, status_block, stream);
    if (error != cudaSuccess) return cuda_fail(error, "peer output addresses");
  } else {
    error = fmoe::launch_route_build(f.topk_ids, routes, f.experts, lists, status_block, counts, offsets, sorted_routes, row_expert, scratch,
                                     stream, reinterpret_cast<int*>(base + layout.route_pos));
    if (error != cudaSuccess) return cuda_fail(error, "route build");
  }
  mark(FMOE_STAGE_ROUTE + 1);
  const int* valid_rows = peer ? f.sorted_offsets + f.experts : offsets + f.experts;
  const void* gemm_rows = base + layout.a_rows;
  const float* gemm_row_scale = a_scale;

  if (peer) {
    gemm_rows = f.x;  // already sorted, already quantised
    gemm_row_scale = f.rows_scale;
  } else if (f.rows_mode && f.int8) {
    // int8 rows travel as H bytes: gather them as H/2 16-bit words, then their scales.
    error = fmoe::launch_gather_rows(static_cast<const uint16_t*>(f.x), routes, f.hidden / 2, sorted_routes, 1, valid_rows,
                                     reinterpret_cast<uint16_t*>(base + layout.a_rows), stream);
    if (error == cudaSuccess) error = fmoe::launch_gather_scalars(f.rows_scale, routes, sorted_routes, valid_rows, a_scale, stream);
  } else if (planes) {
    error = fmoe::launch_split_tokens_scatter_planes(static_cast<const uint16_t*>(f.x), f.tokens, f.hidden, f.top_k,
                                                     reinterpret_cast<const int*>(base + layout.route_pos),
                                                     reinterpret_cast<int8_t*>(base + layout.a_rows), a_scale, stream);
  } else if (f.int8) {
    error = fmoe::launch_quantize_tokens_scatter(static_cast<const uint16_t*>(f.x), f.tokens, f.hidden, f.top_k,
                                                 reinterpret_cast<const int*>(base + layout.route_pos), cfg.numerics,
                                                 reinterpret_cast<int8_t*>(base + layout.a_rows), a_scale, stream);
  } else {
    error = fmoe::launch_gather_rows(static_cast<const uint16_t*>(f.x), routes, f.hidden, sorted_routes, f.top_k, valid_rows,
                                     reinterpret_cast<uint16_t*>(base + layout.a_rows), stream);
  }
  if (error != cudaSuccess) return cuda_fail(error, "activation quantise/gather");
  mark(FMOE_STAGE_QUANT_IN + 1);

  fmoe::GroupedGemmArgs gu;
  memset(&gu, 0, sizeof(gu));
  gu.a_rows = gemm_rows;
  gu.weights = f.w13;
  gu.a_scale = gemm_row_scale;
  gu.w_scale = f.s13;
  gu.items = items_gu;
  gu.status = status_block;
  gu.status_rw = status_block;
  gu.item_count_word = fmoe::kStatusItems;
  gu.max_items = max_items;
  gu.sorted_routes = sorted_routes;
  gu.experts = f.experts;
  gu.k = f.hidden;
  gu.n_out = f.inter;
  gu.numerics = cfg.numerics;
  gu.w8a16 = planes ? 2 : (f.w8a16 ? 1 : 0);
  gu.swiglu_limit = cfg.swiglu_limit;
  gu.activation = cfg.activation;
  gu.expert_bias = cfg.w13_bias;
  gu.y = y;
  gu.route_out = nullptr;
  gu.dump_acc = cfg.dump_acc1;
  gu.total_rows = routes;
  gu.row_tile = (planes && tile_gu != fmoe::kPairRowTile) ? 2 * tile_gu : tile_gu;
  const bool int8_gemm = f.int8 || planes;
#ifdef FMOE_DIAG
  error = umma ? fmoe::launch_umma_grouped_gemm(gu, int8_gemm, true, stream) : fmoe::launch_simt_grouped_gemm(gu, f.int8, true, stream);
#else
  error = fmoe::launch_umma_grouped_gemm(gu, int8_gemm, true, stream);
#endif
  if (error == cudaSuccess && split) {
    fmoe::GroupedGemmArgs big = gu;
    big.items = items_gu_big;
    big.item_count_word = fmoe::kStatusItemsC;
    big.row_tile = fmoe::kPairRowTile;
    error = fmoe::launch_umma_grouped_gemm(big, int8_gemm, true, stream);
  }
  if (error != cudaSuccess) return cuda_fail(error, "gate_up grouped GEMM");
  mark(FMOE_STAGE_GATE_UP + 1);

  const void* down_rows = y;
  if (f.int8) {
    int8_t* yq = reinterpret_cast<int8_t*>(base + layout.yq);
    error = fmoe::launch_quantize_rows(y, routes, f.inter, nullptr, 1, valid_rows, cfg.numerics, 0, yq, y_scale, stream);
    if (error != cudaSuccess) return cuda_fail(error, "intermediate quantise");
    down_rows = yq;
  } else if (planes) {
    int8_t* y_planes = reinterpret_cast<int8_t*>(base + (f.inter > f.hidden ? layout.yq : layout.a_rows));
    error = fmoe::launch_split_rows_planes(y, routes, f.inter, nullptr, 1, valid_rows, y_planes, y_scale, stream);
    if (error != cudaSuccess) return cuda_fail(error, "intermediate planes");
    down_rows = y_planes;
  }
  mark(FMOE_STAGE_QUANT_MID + 1);

  fmoe::GroupedGemmArgs dn = gu;
  dn.a_rows = down_rows;
  dn.weights = f.w2;
  dn.a_scale = y_scale;
  dn.w_scale = f.s2;
  dn.expert_bias = cfg.w2_bias;
  dn.items = items_dn;
  dn.item_count_word = fmoe::kStatusItemsB;
  dn.k = f.inter;
  dn.n_out = f.hidden;
  dn.y = nullptr;
  dn.route_out = route_out;
  dn.row_out_ptrs = row_out_ptrs;
  // bf16 route rows: the peer-memory return in its compact form, or the single-GPU compact mode of fmoe_config.
  const bool compact_rows = peer ? f.peer_rows_bf16 : (cfg.route_rows_bf16 != 0 && !f.rows_mode);
  dn.route_out_bf16 = compact_rows ? 1 : 0;
  dn.dump_acc = cfg.dump_acc2;
  dn.row_tile = (planes && tile_dn != fmoe::kPairRowTile) ? 2 * tile_dn : tile_dn;
#ifdef FMOE_DIAG
  error = umma ? fmoe::launch_umma_grouped_gemm(dn, int8_gemm, false, stream) : fmoe::launch_simt_grouped_gemm(dn, f.int8, false, stream);
#else
  error = fmoe::launch_umma_grouped_gemm(dn, int8_gemm, false, stream);
#endif
  if (error == cudaSuccess && split) {
    fmoe::GroupedGemmArgs big = dn;
    big.items = items_dn_big;
    big.item_count_word = fmoe::kStatusItemsD;
    big.row_tile = fmoe::kPairRowTile;
    error = fmoe::launch_umma_grouped_gemm(big, int8_gemm, false, stream);
  }
  if (error != cudaSuccess) return cuda_fail(error, "down grouped GEMM");
  mark(FMOE_STAGE_DOWN + 1);

  if (!f.rows_mode && compact_rows) {
    error = fmoe::launch_merge_bf16_rows(reinterpret_cast<const uint16_t*>(route_out), f.topk_weights, f.tokens, f.top_k, f.hidden,
                                         f.int8 ? 0 : 1, static_cast<uint16_t*>(out), stream, reinterpret_cast<const int*>(base + layout.route_pos));
    if (error != cudaSuccess) return cuda_fail(error, "top-k merge");
  } else if (!f.rows_mode) {
    error = fmoe::launch_merge(route_out, f.topk_weights, f.tokens, f.top_k, f.hidden, f.int8 ? 0 : 1, static_cast<uint16_t*>(out), stream,
                               reinterpret_cast<const int*>(base + layout.route_pos));
    if (error != cudaSuccess) return cuda_fail(error, "top-k merge");
  }
  mark(FMOE_STAGE_MERGE + 1);
  return FMOE_OK;
}

}  // namespace

namespace fmoe {
// Lets entry points defined in other translation units set the thread's error text.
int report_error(int code, const char* text) { return fail(code, "%s", text); }
}  // namespace fmoe

extern "C" {

int fmoe_abi_version(void) { return FMOE_ABI_VERSION; }

const char* fmoe_last_error(void) { return g_error; }

int fmoe_device_supported(int device) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}

int fmoe_read_status(const void* workspace, void* stream, int32_t* error, int32_t* detail) {
  if (workspace == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "workspace is null");
  int words[fmoe::kStatusWords];
  cudaError_t result = cudaMemcpyAsync(words, workspace, sizeof(words), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (result == cudaSuccess) result = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (result != cudaSuccess) return cuda_fail(result, "reading the status block");
  if (error) *error = words[fmoe::kStatusError];
  if (detail) *detail = words[fmoe::kStatusDetail];
  if (words[fmoe::kStatusError] == FMOE_ERR_EXPERT_ID_RANGE) {
    fail(FMOE_ERR_EXPERT_ID_RANGE, "topk expert id is out of range at flat route %d", words[fmoe::kStatusDetail]);
  } else if (words[fmoe::kStatusError] == FMOE_ERR_DEVICE_WAIT) {
    if (words[fmoe::kStatusWaitSite] != 0) {
      fail(FMOE_ERR_DEVICE_WAIT, "a bounded device wait gave up (CTA %d, site %d)", words[fmoe::kStatusDetail],
           words[fmoe::kStatusWaitSite]);
    } else if (words[fmoe::kStatusDetail] >= 0) {
      fail(FMOE_ERR_DEVICE_WAIT, "a peer barrier gave up waiting for rank %d", words[fmoe::kStatusDetail]);
    } else {
      fail(FMOE_ERR_DEVICE_WAIT, "an expert-parallel row carried an invalid destination or return address (check %d)",
           -words[fmoe::kStatusDetail]);
    }
  }
  return FMOE_OK;
}

int fmoe_stage_timer_create(int32_t max_calls, void** timer) {
  if (timer == nullptr || max_calls <= 0 || max_calls > 4096) return fail(FMOE_ERR_INVALID_ARGUMENT, "invalid stage timer request");
  StageTimer* created = new StageTimer();
  created->max_calls = max_calls;
  created->events.resize(static_cast<size_t>(max_calls) * (FMOE_STAGES + 1));
  for (cudaEvent_t& event : created->events) {
    const cudaError_t error = cudaEventCreate(&event);
    if (error != cudaSuccess) return cuda_fail(error, "cudaEventCreate");
  }
  *timer = created;
  return FMOE_OK;
}

int fmoe_stage_timer_destroy(void* timer) {
  StageTimer* owned = static_cast<StageTimer*>(timer);
  if (owned == nullptr) return FMOE_OK;
  for (cudaEvent_t event : owned->events) cudaEventDestroy(event);
  delete owned;
  return FMOE_OK;
}

int fmoe_stage_timer_reset(void* timer) {
  if (timer == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "timer is null");
  static_cast<StageTimer*>(timer)->calls = 0;
  return FMOE_OK;
}

int fmoe_stage_timer_calls(void* timer) { return timer == nullptr ? 0 : static_cast<StageTimer*>(timer)->calls; }

int fmoe_stage_timer_read(void* timer, int32_t call, float* stage_ms) {
  StageTimer* owned = static_cast<StageTimer*>(timer);
  if (owned == nullptr || stage_ms == nullptr || call < 0 || call >= owned->calls) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "invalid stage timer read");
  }
  cudaEvent_t* marks = owned->events.data() + static_cast<size_t>(call) * (FMOE_STAGES + 1);
  cudaError_t error = cudaEventSynchronize(marks[FMOE_STAGES]);
  if (error != cudaSuccess) return cuda_fail(error, "cudaEventSynchronize");
  for (int stage = 0; stage < FMOE_STAGES; ++stage) {
    error = cudaEventElapsedTime(stage_ms + stage, marks[stage], marks[stage + 1]);
    if (error != cudaSuccess) return cuda_fail(error, "cudaEventElapsedTime");
  }
  return FMOE_OK;
}

int fmoe_w8a8_workspace_layout(int64_t tokens, int32_t top_k, int32_t experts, int32_t hidden, int32_t inter,
                               fmoe_workspace_layout* layout) {
  return make_layout(true, tokens, top_k, experts, hidden, inter, layout);
}

int fmoe_bf16_workspace_layout(int64_t tokens, int32_t top_k, int32_t experts, int32_t hidden, int32_t inter,
                               fmoe_workspace_layout* layout) {
  return make_layout(false, tokens, top_k, experts, hidden, inter, layout);
}

int fmoe_w8a8_forward(const void* x, const int8_t* w13, const float* s13, const int8_t* w2, const float* s2,
                      const float* topk_weights, const int64_t* topk_ids, int64_t tokens, int32_t top_k,
                      int32_t experts, int32_t hidden, int32_t inter, const fmoe_config* config, void* out,
                      void* workspace, size_t workspace_bytes, void* stream) {
  const Forward f{true, x, w13, s13, w2, s2, topk_weights, topk_ids, tokens, top_k, experts, hidden, inter};
  return run_forward(f, config, out, workspace, workspace_bytes, stream);
}

int fmoe_bf16_forward(const void* x, const void* w13, const void* w2, const float* topk_weights,
                      const int64_t* topk_ids, int64_t tokens, int32_t top_k, int32_t experts, int32_t hidden,
                      int32_t inter, const fmoe_config* config, void* out, void* workspace, size_t workspace_bytes,
                      void* stream) {
  const Forward f{false, x, w13, nullptr, w2, nullptr, topk_weights, topk_ids, tokens, top_k, experts, hidden, inter};
  return run_forward(f, config, out, workspace, workspace_bytes, stream);
}

int fmoe_w8a16_forward(const void* x, const int8_t* w13, const float* s13, const int8_t* w2, const float* s2, const float* topk_weights,
                       const int64_t* topk_ids, int64_t tokens, int32_t top_k, int32_t experts, int32_t hidden, int32_t inter,
                       const fmoe_config* config, void* out, void* workspace, size_t workspace_bytes, void* stream) {
  Forward f{false, x, w13, s13, w2, s2, topk_weights, topk_ids, tokens, top_k, experts, hidden, inter};
  f.w8a16 = true;
#ifdef FMOE_DIAG
  if (config != nullptr && config->gemm_impl == FMOE_GEMM_SIMT) return fail(FMOE_ERR_INVALID_ARGUMENT, "W8A16 runs on the tensor-core GEMM only");
#endif
  return run_forward(f, config, out, workspace, workspace_bytes, stream);
}

int fmoe_w8a8_expert_rows_forward(const int8_t* rows_q, const float* rows_scale, const int64_t* rows_expert, int64_t rows,
                                  const int8_t* w13, const float* s13, const int8_t* w2, const float* s2, int32_t experts,
                                  int32_t hidden, int32_t inter, const fmoe_config* config, float* route_out, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  Forward f{true, rows_q, w13, s13, w2, s2, nullptr, rows_expert, rows, 1, experts, hidden, inter};
  f.rows_scale = rows_scale;
  f.route_out_override = route_out;
  f.rows_mode = true;
  return run_forward(f, config, nullptr, workspace, workspace_bytes, stream);
}

int fmoe_bf16_expert_rows_forward(const void* rows, const int64_t* rows_expert, int64_t row_count, const void* w13, const void* w2,
                                  int32_t experts, int32_t hidden, int32_t inter, const fmoe_config* config, float* route_out,
                                  void* workspace, size_t workspace_bytes, void* stream) {
  Forward f{false, rows, w13, nullptr, w2, nullptr, nullptr, rows_expert, row_count, 1, experts, hidden, inter};
  f.route_out_override = route_out;
  f.rows_mode = true;
  return run_forward(f, config, nullptr, workspace, workspace_bytes, stream);
}

size_t fmoe_ep_dispatch_workspace_bytes(int64_t tokens, int32_t top_k, int32_t world) {
  if (tokens < 0 || top_k <= 0 || world <= 0) return 0;
  const size_t routes = static_cast<size_t>(tokens) * top_k;
  return align_up(sizeof(int) * fmoe::kStatusWords, 256) + align_up(sizeof(int64_t) * (routes > 0 ? routes : 1), 256) +
         align_up(sizeof(int) * (world + 1), 256) + align_up(sizeof(int) * (routes > 0 ? routes : 1), 256) +
         align_up(fmoe::route_scratch_bytes(routes, world), 256) + 256;
}

int fmoe_ep_dispatch_prepare(const void* x, const int64_t* topk_ids, int64_t tokens, int32_t top_k, int32_t experts_global,
                             int32_t world, int32_t shared_rank, int32_t hidden, int32_t int8, int32_t numerics, int32_t* dest_counts,
                             int32_t* send_order, void* send_rows, float* send_scale, int64_t* send_expert, void* workspace,
                             size_t workspace_bytes, void* stream_ptr) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  if (tokens < 0 || top_k <= 0 || top_k > 32 || world <= 0 || world > fmoe::kMaxExperts || experts_global <= 0 ||
      experts_global % world != 0 || hidden <= 0 || hidden % 16 != 0 || shared_rank >= world) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "invalid dispatch shape (experts must divide evenly over the ranks, H %% 16 == 0)");
  }
  if (dest_counts == nullptr || workspace == nullptr || workspace_bytes < fmoe_ep_dispatch_workspace_bytes(tokens, top_k, world)) {
    return fail(FMOE_ERR_WORKSPACE, "dispatch workspace missing or too small");
  }
  const int64_t routes = tokens * top_k;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  char* cursor = static_cast<char*>(workspace);
  auto take = [&cursor](size_t bytes) {
    char* begin = cursor;
    cursor += align_up(bytes, 256);
    return begin;
  };
  int* status_block = reinterpret_cast<int*>(take(sizeof(int) * fmoe::kStatusWords));
  int64_t* dest = reinterpret_cast<int64_t*>(take(sizeof(int64_t) * (routes > 0 ? routes : 1)));
  int* offsets = reinterpret_cast<int*>(take(sizeof(int) * (world + 1)));
  int* row_rank = reinterpret_cast<int*>(take(sizeof(int) * (routes > 0 ? routes : 1)));
  int* scratch = reinterpret_cast<int*>(take(fmoe::route_scratch_bytes(routes, world)));
  cudaError_t error = cudaMemsetAsync(status_block, 0, sizeof(int) * fmoe::kStatusWords, stream);
  if (error != cudaSuccess) return cuda_fail(error, "cudaMemsetAsync(status)");
  if (routes == 0) {
    error = cudaMemsetAsync(dest_counts, 0, sizeof(int) * world, stream);
    return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "cudaMemsetAsync(counts)");
  }
  if (x == nullptr || topk_ids == nullptr || send_order == nullptr || send_rows == nullptr || send_expert == nullptr ||
      (int8 && send_scale == nullptr)) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "null pointer");
  }
  error = fmoe::launch_dest_ranks(topk_ids, routes, experts_global, experts_global / world, shared_rank, dest, stream);
  if (error == cudaSuccess) {
    // A stable counting sort of the routes by destination rank: the same kernels as the per-expert route build.
    error = fmoe::launch_route_build(dest, routes, world, fmoe::no_item_lists(), status_block, dest_counts, offsets, send_order, row_rank,
                                     scratch, stream);
  }
  const int* valid_rows = offsets + world;
  if (error == cudaSuccess) {
    if (int8) {
      error = fmoe::launch_quantize_rows(static_cast<const uint16_t*>(x), routes, hidden, send_order, top_k, valid_rows, numerics, 0,
                                         static_cast<int8_t*>(send_rows), send_scale, stream);
    } else {
      error = fmoe::launch_gather_rows(static_cast<const uint16_t*>(x), routes, hidden, send_order, top_k, valid_rows,
                                       static_cast<uint16_t*>(send_rows), stream);
    }
  }
  if (error == cudaSuccess) {
    error = fmoe::launch_local_experts(topk_ids, send_order, routes, valid_rows, experts_global, experts_global / world, send_expert, stream);
  }
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "expert-parallel dispatch");
}

int fmoe_ep_combine_finish(const float* returned_rows, const int32_t* send_order, const float* topk_weights, int64_t tokens,
                           int32_t top_k, int32_t hidden, int32_t tree_merge, float* route_out, void* out, void* stream_ptr) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  if (tokens < 0 || top_k <= 0 || top_k > 32 || hidden <= 0 || hidden % 16 != 0) return fail(FMOE_ERR_INVALID_ARGUMENT, "invalid combine shape");
  if (tokens == 0) return FMOE_OK;
  if (returned_rows == nullptr || send_order == nullptr || topk_weights == nullptr || route_out == nullptr || out == nullptr) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "null pointer");
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  cudaError_t error = fmoe::launch_scatter_rows_f32(returned_rows, send_order, tokens * top_k, nullptr, hidden, route_out, stream);
  if (error == cudaSuccess) {
    error = fmoe::launch_merge(route_out, topk_weights, tokens, top_k, hidden, tree_merge, static_cast<uint16_t*>(out), stream);
  }
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "expert-parallel combine");
}

int fmoe_quantize_weight_rows(const void* w, int64_t rows, int32_t cols, int8_t* q, float* scale, void* stream) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  if (rows < 0 || cols <= 0 || cols % 16 != 0) return fail(FMOE_ERR_INVALID_ARGUMENT, "cols must be a positive multiple of 16");
  if (rows > 0 && (w == nullptr || q == nullptr || scale == nullptr)) return fail(FMOE_ERR_INVALID_ARGUMENT, "null pointer");
  const cudaError_t error = fmoe::launch_quantize_rows(static_cast<const uint16_t*>(w), rows, cols, nullptr, 1, nullptr,
                                                       FMOE_NUMERICS_TORCHREF, 1, q, scale, static_cast<cudaStream_t>(stream));
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "weight quantiser");
}

int fmoe_quantize_rows(const void* x, int64_t rows, int32_t cols, int32_t numerics, int8_t* q, float* scale, void* stream) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  if (rows < 0 || cols <= 0 || cols % 16 != 0) return fail(FMOE_ERR_INVALID_ARGUMENT, "cols must be a positive multiple of 16");
  if (numerics != FMOE_NUMERICS_TORCHREF && numerics != FMOE_NUMERICS_NATIVE) return fail(FMOE_ERR_INVALID_ARGUMENT, "unknown numerics");
  if (rows > 0 && (x == nullptr || q == nullptr || scale == nullptr)) return fail(FMOE_ERR_INVALID_ARGUMENT, "null pointer");
  const cudaError_t error = fmoe::launch_quantize_rows(static_cast<const uint16_t*>(x), rows, cols, nullptr, 1, nullptr, numerics, 0, q,
                                                       scale, static_cast<cudaStream_t>(stream));
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "row quantiser");
}

namespace {
struct DenseLayout {
  size_t status, items, xq, scale, total;
  int max_items;
  int k_padded;
};

DenseLayout dense_layout(int64_t rows, int k) {
  DenseLayout d;
  d.k_padded = static_cast<int>(align_up(static_cast<size_t>(k), 16));
  d.max_items = static_cast<int>(rows / 16 + 2);
  size_t offset = 0;
  auto take = [&offset](size_t bytes) {
    const size_t begin = offset;
    offset = align_up(offset + bytes, 256);
    return begin;
  };
  const size_t r = static_cast<size_t>(rows > 0 ? rows : 1);
  d.status = take(sizeof(int) * fmoe::kStatusWords);
  d.items = take(sizeof(int) * 4 * static_cast<size_t>(d.max_items));
  d.xq = take(r * d.k_padded);
  d.scale = take(sizeof(float) * r);
  d.total = offset;
  return d;
}

// Row tile of the dense GEMM: the smallest one-SM tile that holds a decode batch, the two-SM kernel (256-row work
// items) for anything taller than one 128-row tile.
int dense_row_tile(int64_t rows) {
  if (rows <= 16) return 16;
  if (rows <= 32) return 32;
  if (rows <= 64) return 64;
  if (rows <= 128) return 128;
  return fmoe::kPairRowTile;
}

// Split-K for products with very few rows: how many parts the K range of a channel block is cut into so that the work
// units fill the SMs (every part at least two 128-byte K blocks), and the bytes its table of partial sums and its
// counters take behind the base layout.  Such a product is latency-bound (a 7168 x 1536 projection streams 11 MB: 2 us
// of HBM time inside 20 us of launches, prologue and one CTA's 0.9 MB stream); measured in a CUDA graph, per op:
// 1 row 20.2 -> 14.7 us, 16 rows 19.5 -> 15.7 us, but 64 rows 22.4 -> 24.9 us and 128 rows x 16384 x 7168 48.7 -> 64.3 us
// (8192 atomic additions per work unit), hence the row limit.  FUSED_CPP_MOE_DENSE_SPLIT=0 switches it off.
constexpr int kDenseSplitMaxRows = 16;

int dense_split_parts(int64_t rows, int k_padded, int n) {
  if (rows <= 0 || rows > kDenseSplitMaxRows) return 1;
  const char* text = getenv("FUSED_CPP_MOE_DENSE_SPLIT");
  if (text != nullptr && text[0] == '0') return 1;
  const int n_blocks = (n + 127) / 128;
  const int k_blocks = (k_padded + 127) / 128;
  int parts = fmoe::sm_count_of_current_device() / n_blocks;
  if (parts > k_blocks / 2) parts = k_blocks / 2;
  if (parts > 16) parts = 16;
  return parts >= 2 ? parts : 1;
}

size_t dense_split_bytes(int64_t rows, int n, int max_items) {
  if (rows <= 0 || rows > kDenseSplitMaxRows || n <= 0) return 0;
  const size_t n_blocks = static_cast<size_t>((n + 127) / 128);
  return align_up(static_cast<size_t>(rows) * n * sizeof(int), 256) + align_up(sizeof(int) * n_blocks * static_cast<size_t>(max_items), 256);
}

// One int8 GEMM with the dense epilogue over already-quantised rows.
cudaError_t dense_gemm(const DenseLayout& d, char* base, size_t workspace_bytes, int64_t rows, const int8_t* w, const float* w_scale,
                       const float* bias, int n, void* out, int out_is_bf16, int row_tile, cudaStream_t stream) {
  fmoe::GroupedGemmArgs args;
  memset(&args, 0, sizeof(args));
  const int parts = dense_split_parts(rows, d.k_padded, n);
  const size_t split_bytes = dense_split_bytes(rows, n, d.max_items);
  if (parts > 1 && workspace_bytes >= d.total + split_bytes) {
    // Partial sums and counters start at zero (one memset: the two regions are adjacent).
    const cudaError_t error = cudaMemsetAsync(base + d.total, 0, split_bytes, stream);
    if (error != cudaSuccess) return error;
    args.dense_splits = parts;
    args.dense_partial = reinterpret_cast<int*>(base + d.total);
    args.dense_counters = reinterpret_cast<int*>(base + d.total + align_up(static_cast<size_t>(rows) * n * sizeof(int), 256));
  }
  args.a_rows = base + d.xq;
  args.weights = w;
  args.a_scale = reinterpret_cast<const float*>(base + d.scale);
  args.w_scale = w_scale;
  args.items = reinterpret_cast<const int*>(base + d.items);
  args.status = reinterpret_cast<const int*>(base + d.status);
  args.status_rw = reinterpret_cast<int*>(base + d.status);
  args.item_count_word = fmoe::kStatusItems;
  args.max_items = d.max_items;
  args.experts = 1;
  args.k = d.k_padded;
  args.n_out = n;
  args.numerics = FMOE_NUMERICS_TORCHREF;  // (acc * x_scale) * w_scale, csrc/i8gemm.cpp:157
  args.total_rows = rows;
  args.row_tile = row_tile;
  args.dense_out = out;
  args.dense_out_bf16 = out_is_bf16;
  args.bias = bias;
  return fmoe::launch_umma_grouped_gemm(args, true, false, stream);
}

int dense_prologue(const void* x, int x_is_bf16, int64_t rows, int k, int clamp_low, void* workspace, size_t workspace_bytes,
                   DenseLayout* layout, int* row_tile, cudaStream_t stream) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  if (rows < 0 || k <= 0) return fail(FMOE_ERR_INVALID_ARGUMENT, "i8gemm: rows must be >= 0 and K positive");
  *layout = dense_layout(rows, k);
  if (rows == 0) return FMOE_OK;
  if (x == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "i8gemm: null input");
  if (workspace == nullptr || workspace_bytes < layout->total || reinterpret_cast<uintptr_t>(workspace) % 256 != 0) {
    return fail(FMOE_ERR_WORKSPACE, "i8gemm: workspace missing, misaligned or too small (%zu bytes needed)", layout->total);
  }
  char* base = static_cast<char*>(workspace);
  *row_tile = dense_row_tile(rows);
  // One launch: the quantiser's first block also resets the status block and writes the GEMM's work items.
  const cudaError_t error = fmoe::launch_quantize_rows_dense(
      x, x_is_bf16, rows, k, layout->k_padded, clamp_low, reinterpret_cast<int8_t*>(base + layout->xq),
      reinterpret_cast<float*>(base + layout->scale), *row_tile == fmoe::kPairRowTile ? 256 : *row_tile, layout->max_items,
      reinterpret_cast<int*>(base + layout->items), reinterpret_cast<int*>(base + layout->status), stream);
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "i8gemm activation quantisation");
}
}  // namespace

size_t fmoe_i8gemm_workspace_bytes(int64_t rows, int32_t k, int32_t n) {
  if (rows < 0 || k <= 0) return 0;
  const DenseLayout layout = dense_layout(rows, k);
  return layout.total + dense_split_bytes(rows, n, layout.max_items);  // n = the widest product that will use the workspace
}

int fmoe_i8gemm_dynamic_scaled_mm(const void* x, int32_t x_is_bf16, int64_t rows, int32_t k, const int8_t* w,
                                  const float* w_scale, const float* bias, int32_t n, void* out, int32_t out_is_bf16,
                                  void* workspace, size_t workspace_bytes, void* stream_ptr) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  DenseLayout layout;
  int row_tile = 16;
  if (n <= 0) return fail(FMOE_ERR_INVALID_ARGUMENT, "i8gemm: N must be positive");
  const int status = dense_prologue(x, x_is_bf16, rows, k, -128, workspace, workspace_bytes, &layout, &row_tile, stream);
  if (status != FMOE_OK || rows == 0) return status;
  if (w == nullptr || w_scale == nullptr || out == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "i8gemm: null pointer");
  const cudaError_t error = dense_gemm(layout, static_cast<char*>(workspace), workspace_bytes, rows, w, w_scale, bias, n, out, out_is_bf16, row_tile, stream);
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "i8gemm GEMM");
}

int fmoe_i8gemm_dynamic_scaled_mm_pair(const void* x_bf16, int64_t rows, int32_t k, const int8_t* first_w, const float* first_scale,
                                       int32_t first_n, void* first_out, const int8_t* second_w, const float* second_scale,
                                       int32_t second_n, void* second_out, void* workspace, size_t workspace_bytes,
                                       void* stream_ptr) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  DenseLayout layout;
  int row_tile = 16;
  if (first_n <= 0 || second_n <= 0) return fail(FMOE_ERR_INVALID_ARGUMENT, "i8gemm pair: N must be positive");
  const int status = dense_prologue(x_bf16, 1, rows, k, -127, workspace, workspace_bytes, &layout, &row_tile, stream);
  if (status != FMOE_OK || rows == 0) return status;
  if (first_w == nullptr || second_w == nullptr || first_scale == nullptr || second_scale == nullptr || first_out == nullptr ||
      second_out == nullptr) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "i8gemm pair: null pointer");
  }
  char* base = static_cast<char*>(workspace);
  cudaError_t error = dense_gemm(layout, base, workspace_bytes, rows, first_w, first_scale, nullptr, first_n, first_out, 1, row_tile, stream);
  if (error == cudaSuccess) error = dense_gemm(layout, base, workspace_bytes, rows, second_w, second_scale, nullptr, second_n, second_out, 1, row_tile, stream);
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "i8gemm pair GEMM");
}

#ifdef FMOE_DIAG
int fmoe_probe_mma_rate(int32_t int8, int32_t n, int32_t iterations, int32_t mode, float* tera_ops_per_s) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  // The iteration cap keeps one launch (about 0.1 us per MMA at n = 256) far below the kernels' one-second wait limit.
  if ((mode & 16) && (mode >> 8) <= 0) return fail(FMOE_ERR_INVALID_ARGUMENT, "probe: the round-trip mode needs c = mode >> 8 > 0");
  if ((mode & 16) && iterations > 100000) iterations = 100000;  // a round trip is microseconds, not tens of nanoseconds
  if (tera_ops_per_s == nullptr || iterations <= 0 || iterations > 1000000 || n < 16 || n > 256 || n % 16 != 0) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "probe: n must be a multiple of 16 in [16, 256] and iterations in 1..1000000");
  }
  int device = 0, sms = 0;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  int* status_block = nullptr;
  cudaEvent_t begin = nullptr, end = nullptr;
  cudaError_t error = cudaMalloc(&status_block, sizeof(int) * fmoe::kStatusWords);
  if (error == cudaSuccess) error = cudaMemset(status_block, 0, sizeof(int) * fmoe::kStatusWords);
  if (error == cudaSuccess) error = cudaEventCreate(&begin);
  if (error == cudaSuccess) error = cudaEventCreate(&end);
  float best_ms = 0.0f;
  for (int round = 0; round < 4 && error == cudaSuccess; ++round) {
    cudaEventRecord(begin, nullptr);
    error = (mode & 8) ? fmoe::launch_mma_rate_pair_probe(int8 != 0, n, iterations, mode & ~8, sms, status_block, nullptr)
                       : fmoe::launch_mma_rate_probe(int8 != 0, n, iterations, mode, sms, status_block, nullptr);
    cudaEventRecord(end, nullptr);
    if (error == cudaSuccess) error = cudaEventSynchronize(end);
    float ms = 0.0f;
    if (error == cudaSuccess) error = cudaEventElapsedTime(&ms, begin, end);
    if (round > 0 && (best_ms == 0.0f || ms < best_ms)) best_ms = ms;
  }
  if (begin) cudaEventDestroy(begin);
  if (end) cudaEventDestroy(end);
  if (status_block) cudaFree(status_block);
  if (error != cudaSuccess) return cuda_fail(error, "MMA rate probe");
  const double elements_k = int8 ? 32.0 : 16.0;
  // One-SM MMAs: 128 x n per SM; two-SM MMAs (mode bit 3): 256 x n per pair of SMs.
  const double ops = 2.0 * 128.0 * n * elements_k * static_cast<double>(iterations) * ((mode & 8) ? (sms & ~1) : sms);
  *tera_ops_per_s = static_cast<float>(ops / (best_ms * 1e-3) / 1e12);
  return FMOE_OK;
}
#endif  // FMOE_DIAG

}  // extern "C"

extern "C" int fmoe_router_topk(const float* logits, const float* selection_bias, int64_t tokens, int32_t experts, int32_t top_k,
                                int32_t scoring, int32_t renormalize, float routed_scaling_factor, float* topk_weights,
                                int64_t* topk_ids, void* stream) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  if (tokens < 0 || experts <= 0 || experts > fmoe::kMaxExperts || top_k <= 0 || top_k > 32 || top_k > experts) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "router: experts in 1..%d and top_k in 1..min(32, experts) (got %d, %d)", fmoe::kMaxExperts,
                experts, top_k);
  }
  if (scoring != FMOE_SCORING_SOFTMAX && scoring != FMOE_SCORING_SIGMOID) return fail(FMOE_ERR_INVALID_ARGUMENT, "router: unknown scoring %d", scoring);
  if (tokens == 0) return FMOE_OK;
  if (logits == nullptr || topk_weights == nullptr || topk_ids == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "router: null pointer");
  const cudaError_t error = fmoe::launch_router_topk(logits, selection_bias, tokens, experts, top_k, scoring == FMOE_SCORING_SIGMOID,
                                                     renormalize != 0, routed_scaling_factor, topk_weights, topk_ids,
                                                     static_cast<cudaStream_t>(stream));
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "router top-k");
}

/* ---- expert parallelism over peer memory ---------------------------------------------------------- */

struct fmoe_ep_peer_context {
  int world = 0, rank = 0, top_k = 0, hidden = 0, inter = 0, local_experts = 0, int8 = 0, rows_bf16 = 0;
  int64_t tokens_max = 0, capacity = 0;
  fmoe::PeerSlabLayout slab{};
  char* slab_base = nullptr;          // this rank's slab (cudaMalloc, exported by IPC handle)
  std::vector<void*> opened;          // peers' slabs as mapped here (null for this rank)
  uint64_t* peer_slabs_dev = nullptr; // [world] device table of slab addresses
  bool connected = false;
  // Local scratch of the dispatch and of the expert stage.
  char* dispatch_ws = nullptr;
  size_t dispatch_ws_bytes = 0;
  char* expert_ws = nullptr;
  size_t expert_ws_bytes = 0;
  int experts_total_max = 0;          // routed experts of all ranks + 1: row length of the count table in the slab
  char* scrap_row = nullptr;          // device: one result row that absorbs stores of rows without a valid return address
  int* small = nullptr;               // device: send_base[experts_total_max] | local_counts[local] | local_offsets[local+1] | epoch
  int* send_base = nullptr;
  int* local_counts = nullptr;
  int* local_offsets = nullptr;
  unsigned* epoch = nullptr;          // [1] barrier epoch of this rank
  unsigned long long wait_limit_ns = 5000000000ull;  // bound of the barrier wait (FUSED_CPP_MOE_EP_WAIT_MS)
};

namespace {

struct DispatchScratch {
  int* status;
  int* counts;      // [experts_total] routes of this rank per global expert
  int* offsets;     // [experts_total + 1]
  int* send_order;  // [routes] flat route ids in expert order
  int* row_expert;  // [routes]
  int* route_pos;   // [routes] position of every flat route in that order, -1 = dropped
  int* scratch;
};

size_t dispatch_scratch_bytes(int64_t routes, int experts_total) {
  const size_t r = static_cast<size_t>(routes > 0 ? routes : 1);
  return align_up(sizeof(int) * fmoe::kStatusWords, 256) + align_up(sizeof(int) * experts_total, 256) +
         align_up(sizeof(int) * (experts_total + 1), 256) + 3 * align_up(sizeof(int) * r, 256) +
         align_up(fmoe::route_scratch_bytes(routes, experts_total), 256);
}

DispatchScratch carve_dispatch(char* base, int64_t routes, int experts_total) {
  const size_t r = static_cast<size_t>(routes > 0 ? routes : 1);
  char* cursor = base;
  auto take = [&cursor](size_t bytes) {
    char* begin = cursor;
    cursor += align_up(bytes, 256);
    return begin;
  };
  DispatchScratch d;
  d.status = reinterpret_cast<int*>(take(sizeof(int) * fmoe::kStatusWords));
  d.counts = reinterpret_cast<int*>(take(sizeof(int) * experts_total));
  d.offsets = reinterpret_cast<int*>(take(sizeof(int) * (experts_total + 1)));
  d.send_order = reinterpret_cast<int*>(take(sizeof(int) * r));
  d.row_expert = reinterpret_cast<int*>(take(sizeof(int) * r));
  d.route_pos = reinterpret_cast<int*>(take(sizeof(int) * r));
  d.scratch = reinterpret_cast<int*>(take(fmoe::route_scratch_bytes(routes, experts_total)));
  return d;
}

}  // namespace

extern "C" {

int fmoe_ep_peer_create(int32_t world, int32_t rank, int64_t tokens_max, int32_t top_k, int32_t hidden, int32_t inter,
                        int32_t local_experts, int32_t int8, int32_t return_bf16, fmoe_ep_peer_context** out) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  if (out == nullptr || world <= 0 || world > 64 || rank < 0 || rank >= world || tokens_max <= 0 || top_k <= 0 || top_k > 32 ||
      local_experts <= 0) {
    return fail(FMOE_ERR_INVALID_ARGUMENT, "invalid peer context shape");
  }
  status = check_shape(tokens_max, top_k, local_experts, hidden, inter);
  if (status != FMOE_OK) return status;
  fmoe_ep_peer_context* ctx = new fmoe_ep_peer_context();
  ctx->world = world;
  ctx->rank = rank;
  ctx->top_k = top_k;
  ctx->hidden = hidden;
  ctx->inter = inter;
  ctx->local_experts = local_experts;
  ctx->int8 = int8 ? 1 : 0;
  ctx->rows_bf16 = return_bf16 ? 1 : 0;
  ctx->tokens_max = tokens_max;
  // Worst case: every route of every rank lands here.
  ctx->capacity = static_cast<int64_t>(world) * tokens_max * top_k;
  const size_t capacity = static_cast<size_t>(ctx->capacity);
  size_t offset = 0;
  auto take = [&offset](size_t bytes) {
    const size_t begin = offset;
    offset = align_up(offset + bytes, 256);
    return begin;
  };
  ctx->experts_total_max = world * local_experts + 1;
  if (ctx->experts_total_max > fmoe::kMaxExperts) {
    delete ctx;
    return fail(FMOE_ERR_INVALID_ARGUMENT, "too many experts for the peer context (%d)", world * local_experts);
  }
  ctx->slab.rows = take(capacity * hidden * (int8 ? 1 : 2));
  ctx->slab.scale = take(capacity * sizeof(float));
  ctx->slab.source = take(capacity * 2 * sizeof(int));
  ctx->slab.route_out = take(static_cast<size_t>(tokens_max) * top_k * hidden * sizeof(float));
  ctx->slab.counts = take(sizeof(int) * static_cast<size_t>(world) * ctx->experts_total_max);
  ctx->slab.flags = take(sizeof(unsigned) * world);
  ctx->slab.total = offset;
  if (const char* limit = getenv("FUSED_CPP_MOE_EP_WAIT_MS")) {
    const long long ms = atoll(limit);
    if (ms > 0) ctx->wait_limit_ns = static_cast<unsigned long long>(ms) * 1000000ull;
  }
  fmoe_workspace_layout layout;
  status = make_layout(int8 != 0, ctx->capacity, 1, local_experts, hidden, inter, &layout, false);
  if (status != FMOE_OK) {
    delete ctx;
    return status;
  }
  ctx->expert_ws_bytes = layout.total_bytes;
  ctx->dispatch_ws_bytes = dispatch_scratch_bytes(tokens_max * top_k, ctx->experts_total_max);
  cudaError_t error = cudaMalloc(&ctx->slab_base, ctx->slab.total);
  if (error == cudaSuccess) error = cudaMalloc(&ctx->expert_ws, ctx->expert_ws_bytes);
  if (error == cudaSuccess) error = cudaMalloc(&ctx->dispatch_ws, ctx->dispatch_ws_bytes);
  if (error == cudaSuccess) error = cudaMalloc(&ctx->peer_slabs_dev, sizeof(uint64_t) * world);
  const size_t small_ints = static_cast<size_t>(ctx->experts_total_max) + local_experts + (local_experts + 1) + 1;
  if (error == cudaSuccess) error = cudaMalloc(&ctx->small, sizeof(int) * small_ints);
  if (error == cudaSuccess) error = cudaMemset(ctx->small, 0, sizeof(int) * small_ints);
  if (error == cudaSuccess) error = cudaMalloc(&ctx->scrap_row, static_cast<size_t>(hidden) * sizeof(float));
  // The whole slab starts at zero: counts and flags must, and a row that is read before it ever arrived (after a
  // barrier that gave up) then carries the return address (rank 0, route 0) and zero data instead of whatever the
  // allocation held.
  if (error == cudaSuccess) error = cudaMemset(ctx->slab_base, 0, ctx->slab.total);
  if (error != cudaSuccess) {
    fmoe_ep_peer_destroy(ctx);
    return cuda_fail(error, "peer context allocation");
  }
  ctx->send_base = ctx->small;
  ctx->local_counts = ctx->send_base + ctx->experts_total_max;
  ctx->local_offsets = ctx->local_counts + local_experts;
  ctx->epoch = reinterpret_cast<unsigned*>(ctx->local_offsets + local_experts + 1);
  ctx->opened.assign(world, nullptr);
  *out = ctx;
  return FMOE_OK;
}

int fmoe_ep_peer_handle(fmoe_ep_peer_context* ctx, void* handle64) {
  if (ctx == nullptr || handle64 == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t handle;
  const cudaError_t error = cudaIpcGetMemHandle(&handle, ctx->slab_base);
  if (error != cudaSuccess) return cuda_fail(error, "cudaIpcGetMemHandle");
  memcpy(handle64, &handle, sizeof(handle));
  return FMOE_OK;
}

int fmoe_ep_peer_connect(fmoe_ep_peer_context* ctx, const void* handles) {
  if (ctx == nullptr || (handles == nullptr && ctx->world > 1)) return fail(FMOE_ERR_INVALID_ARGUMENT, "null pointer");
  if (ctx->connected) return fail(FMOE_ERR_INVALID_ARGUMENT, "peer context is already connected");
  std::vector<uint64_t> table(ctx->world, 0);
  for (int r = 0; r < ctx->world; ++r) {
    if (r == ctx->rank) {
      table[r] = reinterpret_cast<uint64_t>(ctx->slab_base);
      continue;
    }
    cudaIpcMemHandle_t handle;
    memcpy(&handle, static_cast<const char*>(handles) + static_cast<size_t>(r) * sizeof(handle), sizeof(handle));
    void* mapped = nullptr;
    const cudaError_t error = cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess);
    if (error != cudaSuccess) return cuda_fail(error, "cudaIpcOpenMemHandle");
    ctx->opened[r] = mapped;
    table[r] = reinterpret_cast<uint64_t>(mapped);
  }
  const cudaError_t error = cudaMemcpy(ctx->peer_slabs_dev, table.data(), sizeof(uint64_t) * ctx->world, cudaMemcpyHostToDevice);
  if (error != cudaSuccess) return cuda_fail(error, "peer table upload");
  ctx->connected = true;
  return FMOE_OK;
}

void* fmoe_ep_peer_slab_address(fmoe_ep_peer_context* ctx) { return ctx ? ctx->slab_base : nullptr; }

int fmoe_ep_peer_connect_addresses(fmoe_ep_peer_context* ctx, const void* const* slabs) {
  if (ctx == nullptr || slabs == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "null pointer");
  if (ctx->connected) return fail(FMOE_ERR_INVALID_ARGUMENT, "peer context is already connected");
  std::vector<uint64_t> table(ctx->world, 0);
  for (int r = 0; r < ctx->world; ++r) {
    table[r] = r == ctx->rank ? reinterpret_cast<uint64_t>(ctx->slab_base) : reinterpret_cast<uint64_t>(slabs[r]);
    if (table[r] == 0 || table[r] % 256 != 0) return fail(FMOE_ERR_INVALID_ARGUMENT, "slab address of rank %d is null or misaligned", r);
  }
  const cudaError_t error = cudaMemcpy(ctx->peer_slabs_dev, table.data(), sizeof(uint64_t) * ctx->world, cudaMemcpyHostToDevice);
  if (error != cudaSuccess) return cuda_fail(error, "peer table upload");
  ctx->connected = true;
  return FMOE_OK;
}

void fmoe_ep_peer_destroy(fmoe_ep_peer_context* ctx) {
  if (ctx == nullptr) return;
  for (void* mapped : ctx->opened) {
    if (mapped != nullptr) cudaIpcCloseMemHandle(mapped);
  }
  if (ctx->slab_base) cudaFree(ctx->slab_base);
  if (ctx->expert_ws) cudaFree(ctx->expert_ws);
  if (ctx->dispatch_ws) cudaFree(ctx->dispatch_ws);
  if (ctx->peer_slabs_dev) cudaFree(ctx->peer_slabs_dev);
  if (ctx->small) cudaFree(ctx->small);
  if (ctx->scrap_row) cudaFree(ctx->scrap_row);
  delete ctx;
}

int64_t fmoe_ep_peer_slab_bytes(const fmoe_ep_peer_context* ctx) { return ctx ? static_cast<int64_t>(ctx->slab.total) : 0; }

int fmoe_ep_peer_dispatch(fmoe_ep_peer_context* ctx, const void* x, const int64_t* topk_ids, int64_t tokens, int32_t experts_global,
                          int32_t shared_rank, int32_t numerics, void* stream_ptr) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  if (ctx == nullptr || !ctx->connected) return fail(FMOE_ERR_INVALID_ARGUMENT, "peer context missing or not connected");
  const int has_shared = shared_rank >= 0 ? 1 : 0;
  if (tokens < 0 || tokens > ctx->tokens_max || experts_global <= 0 || experts_global % ctx->world != 0 ||
      experts_global / ctx->world + has_shared != ctx->local_experts || (has_shared && shared_rank != ctx->rank) ||
      (tokens > 0 && (x == nullptr || topk_ids == nullptr))) {
    return fail(FMOE_ERR_INVALID_ARGUMENT,
                "invalid peer dispatch arguments (tokens within the context's maximum, experts split evenly and matching the context's "
                "local experts, shared_rank = this rank or -1)");
  }
  if (numerics != FMOE_NUMERICS_TORCHREF && numerics != FMOE_NUMERICS_NATIVE) return fail(FMOE_ERR_INVALID_ARGUMENT, "unknown numerics");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const int64_t routes = tokens * ctx->top_k;
  const int experts_total = experts_global + has_shared;
  const int per_rank = experts_global / ctx->world;
  const DispatchScratch d = carve_dispatch(ctx->dispatch_ws, ctx->tokens_max * ctx->top_k, ctx->experts_total_max);
  cudaError_t error = cudaMemsetAsync(d.status, 0, sizeof(int) * fmoe::kStatusWords, stream);
  if (error == cudaSuccess && routes == 0) error = cudaMemsetAsync(d.counts, 0, sizeof(int) * experts_total, stream);
  if (error == cudaSuccess && routes > 0) {
    // Stable counting sort of this rank's routes by global expert id (the shared expert is id experts_global):
    // expert order is destination-rank order, and inside a destination its local expert order.
    error = fmoe::launch_route_build(topk_ids, routes, experts_total, fmoe::no_item_lists(), d.status, d.counts, d.offsets, d.send_order,
                                     d.row_expert, d.scratch, stream, d.route_pos);
  }
  if (error == cudaSuccess) {
    // Every rank learns every rank's counts per expert (row `rank` of the table in each slab) ...
    error = fmoe::launch_peer_barrier(ctx->peer_slabs_dev, ctx->slab, d.counts, ctx->experts_total_max, ctx->world, ctx->rank, ctx->epoch,
                                      d.status, ctx->wait_limit_ns, stream);
  }
  if (error == cudaSuccess) {
    // ... and derives from them where its rows go and what it will receive.
    error = fmoe::launch_peer_layout(reinterpret_cast<const int*>(ctx->slab_base + ctx->slab.counts), ctx->world, ctx->rank, experts_global,
                                     per_rank, has_shared, ctx->experts_total_max, ctx->send_base, ctx->local_counts, ctx->local_offsets,
                                     d.status, stream);
  }
  if (error == cudaSuccess) {
    error = fmoe::launch_peer_dispatch(ctx->int8 != 0, static_cast<const uint16_t*>(x), topk_ids, tokens, ctx->hidden, ctx->top_k,
                                       d.route_pos, d.offsets, ctx->send_base, ctx->slab, ctx->peer_slabs_dev, ctx->rank, experts_global,
                                       per_rank, has_shared, numerics, ctx->capacity, d.status, stream);
  }
  if (error == cudaSuccess) {
    // After this barrier every row of this rank's experts has arrived.  If it (or the first one) gave up, the
    // counts of this rank's experts are cleared: the expert stage then finds no rows, makes no work items and
    // stores nothing, instead of multiplying rows that are not there.  Every index the later stages derive from
    // the counts stays below `capacity` either way: send_base and the local offsets are sums of at most
    // world x tokens_max x top_k counts when the table is whole, are all zero when the exchange failed, and the
    // dispatch kernel drops (and reports) any row at or beyond `capacity`.
    error = fmoe::launch_peer_barrier(ctx->peer_slabs_dev, ctx->slab, nullptr, 0, ctx->world, ctx->rank, ctx->epoch, d.status,
                                      ctx->wait_limit_ns, stream, ctx->local_counts, 2 * ctx->local_experts + 1);
  }
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "peer dispatch");
}

int fmoe_ep_peer_experts(fmoe_ep_peer_context* ctx, const void* w13, const float* s13, const void* w2, const float* s2,
                         const fmoe_config* config, void* stream) {
  if (ctx == nullptr || !ctx->connected) return fail(FMOE_ERR_INVALID_ARGUMENT, "peer context missing or not connected");
  Forward f{ctx->int8 != 0, ctx->slab_base + ctx->slab.rows, w13, s13, w2, s2, nullptr, nullptr, ctx->capacity, 1, ctx->local_experts,
            ctx->hidden, ctx->inter};
  f.rows_scale = reinterpret_cast<const float*>(ctx->slab_base + ctx->slab.scale);
  f.rows_mode = true;
  f.sorted_counts = ctx->local_counts;
  f.sorted_offsets = ctx->local_offsets;
  f.rows_source = ctx->slab_base + ctx->slab.source;
  f.peer_slabs = ctx->peer_slabs_dev;
  f.peer_route_out_offset = ctx->slab.route_out;
  f.peer_rows_bf16 = ctx->rows_bf16 != 0;
  f.peer_world = ctx->world;
  f.peer_routes_max = ctx->tokens_max * ctx->top_k;
  f.peer_scrap_row = ctx->scrap_row;
  const int status = run_forward(f, config, nullptr, ctx->expert_ws, ctx->expert_ws_bytes, stream);
  if (status != FMOE_OK) return status;
  // After this barrier every result row of this rank's routes has arrived, and every rank is done reading its slab.
  const cudaError_t error = fmoe::launch_peer_barrier(ctx->peer_slabs_dev, ctx->slab, nullptr, 0, ctx->world, ctx->rank, ctx->epoch,
                                                      reinterpret_cast<int*>(ctx->expert_ws), ctx->wait_limit_ns,
                                                      static_cast<cudaStream_t>(stream));
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "peer barrier");
}

int fmoe_ep_peer_combine(fmoe_ep_peer_context* ctx, const float* topk_weights, int64_t tokens, int32_t tree_merge, void* out,
                         void* stream_ptr) {
  int status = check_device();
  if (status != FMOE_OK) return status;
  if (ctx == nullptr || !ctx->connected) return fail(FMOE_ERR_INVALID_ARGUMENT, "peer context missing or not connected");
  if (tokens < 0 || tokens > ctx->tokens_max) return fail(FMOE_ERR_INVALID_ARGUMENT, "tokens exceed the context's maximum");
  if (tokens == 0) return FMOE_OK;
  if (topk_weights == nullptr || out == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "null pointer");
  const char* rows = ctx->slab_base + ctx->slab.route_out;
  const cudaError_t error =
      ctx->rows_bf16 ? fmoe::launch_merge_bf16_rows(reinterpret_cast<const uint16_t*>(rows), topk_weights, tokens, ctx->top_k, ctx->hidden,
                                                    tree_merge, static_cast<uint16_t*>(out), static_cast<cudaStream_t>(stream_ptr))
                     : fmoe::launch_merge(reinterpret_cast<const float*>(rows), topk_weights, tokens, ctx->top_k, ctx->hidden, tree_merge,
                                          static_cast<uint16_t*>(out), static_cast<cudaStream_t>(stream_ptr));
  return error == cudaSuccess ? FMOE_OK : cuda_fail(error, "peer combine");
}

int fmoe_ep_peer_read_status(fmoe_ep_peer_context* ctx, void* stream, int32_t* dispatch_error, int32_t* expert_error) {
  if (ctx == nullptr || dispatch_error == nullptr || expert_error == nullptr) return fail(FMOE_ERR_INVALID_ARGUMENT, "null pointer");
  // The text of fmoe_last_error() describes the first stage that reported something.
  int32_t detail = 0;
  int status = fmoe_read_status(ctx->expert_ws, stream, expert_error, &detail);
  if (status != FMOE_OK) return status;
  char expert_text[sizeof(g_error)];
  memcpy(expert_text, g_error, sizeof(expert_text));
  status = fmoe_read_status(ctx->dispatch_ws, stream, dispatch_error, &detail);
  if (status != FMOE_OK) return status;
  if (*dispatch_error == FMOE_OK && *expert_error != FMOE_OK) memcpy(g_error, expert_text, sizeof(g_error));
  return FMOE_OK;
}

}  // extern "C"
