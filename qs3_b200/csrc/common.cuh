// Internal declarations shared by the translation units of libqs3moe.so.
#pragma once

#include "../../include/qs3_moe.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

// Context object behind the opaque qsfi_context handle. Field order follows
// upstream qsfi_internal.h:11-20 so that an object built against either
// definition reads the same device ordinal, stream and error record.
struct qsfi_context {
    int32_t device_ordinal;
    cudaStream_t stream;
    void* float_workspace;
    size_t float_workspace_bytes;
    size_t int_workspace_bytes;
    size_t host_int_workspace_bytes;
    uint64_t scratch_generation;
    qsfi_error_info last_error;
};

struct qsfi_moe_plan {
    qsfi_moe_plan_desc desc;
    // Side stream of the whole-layer call, created on first use: the token quantiser and the
    // shared expert run there beside the router chain (fork / join with the three events).
    mutable cudaStream_t side_stream = nullptr;
    mutable cudaEvent_t ev_fork = nullptr, ev_quant = nullptr, ev_shared = nullptr;
    mutable int side_state = 0; // 0 not tried, 1 ready, -1 unavailable
};

namespace qs3 {

constexpr size_t kWorkspaceAlign = 256;
constexpr int kTileM = 128; // rows of one tensor-core tile; expert segments are padded to it

// ---- error plumbing (upstream qsfi_context.cu:10-101) -------------------------
void clear_error(qsfi_error_info* err);
qsfi_status set_error(qsfi_context* ctx, qsfi_status status, qsfi_error_source source,
                      int32_t native_code, const char* fmt, ...);
qsfi_status set_invalid_arg(qsfi_context* ctx, const char* fmt, ...);
qsfi_status set_unsupported(qsfi_context* ctx, const char* fmt, ...);
qsfi_status set_cuda_error(qsfi_context* ctx, cudaError_t err, const char* op);
qsfi_status activate_context(qsfi_context* ctx);
qsfi_status status_from_cuda(cudaError_t err);

// Device-side error word shared by the tensor-core kernels (one per device).
uint32_t* device_error_word();

#if QSFI_ENABLE_CHECKED_VALIDATION
// Checked builds only (upstream qsfi_native_common.h checked-validation flag): a device flag
// that validator kernels raise; `checked_flag_finish` copies it back (one stream sync) and
// returns true when it was raised. The flag lives in the library, nothing is allocated.
int* checked_flag_reset(cudaStream_t stream, cudaError_t* err);
bool checked_flag_finish(cudaStream_t stream, cudaError_t* err);
#endif

// Kernel-launch counter (all kernels of this library) and the optional per-stage
// event recorder behind qs3_moe_profile_begin / qs3_moe_profile_end.
void note_launch(uint32_t n = 1);
enum Stage {
    STAGE_END = 0, STAGE_ROUTER_GEMM = 1, STAGE_ROUTER_TOPK = 2, STAGE_ROUTE_SORT = 3,
    STAGE_GATHER = 4, STAGE_GATE_UP_GEMM = 5, STAGE_DOWN_GEMM = 6, STAGE_SHARED = 7, STAGE_COMBINE = 8
};
void stage_mark(cudaStream_t stream, int stage);
bool stage_recording();

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <typename T> bool contiguous1(const T& t) { return t.stride[0] == 1; }
template <typename T> bool contiguous2(const T& t)
{
    return t.stride[1] == 1 && t.stride[0] == t.shape[1];
}
template <typename T> bool contiguous3(const T& t)
{
    return t.stride[2] == 1 && t.stride[1] == t.shape[2]
        && t.stride[0] == t.shape[1] * t.shape[2];
}

// ---- routing tables -------------------------------------------------------------
// Everything the routed path derives from topk_ids, laid out in the workspace.
struct RouteTables {
    int32_t* counts;       // [E] routes per local expert
    int32_t* indptr;       // [E+1] exclusive scan of counts
    int32_t* pad_indptr;   // [E+1] exclusive scan of counts rounded up to tile_rows
    int32_t* route_rows;   // [R] dense row of a route (-1: expert not local)
    int32_t* route_prows;  // [R] row in the padded layout (-1: expert not local)
    int32_t* row_tokens;   // [R] token of a dense row
    float* row_scales;     // [R] routing weight of a dense row
    int32_t* tile_expert;  // [max_tiles]
    int32_t* tile_row0;    // [max_tiles] first padded row of the tile
    int32_t* tile_nrows;   // [max_tiles] valid rows in the tile
    int32_t* total_tiles;  // [1]
    // 256-row "pair tiles" for the CTA-pair GEMM (128-row plans only, NULL otherwise): an expert with t
    // row tiles gives t / 2 full pairs, listed from index 0 upwards, and t % 2 single (<= 128 rows),
    // listed from index max_tiles - 1 downwards; pair_counts = {full pairs, singles}
    int32_t* pair_expert;  // [max_tiles]
    int32_t* pair_row0;    // [max_tiles] first padded row
    int32_t* pair_nrows;   // [max_tiles] valid rows, 1..256
    int32_t* pair_counts;  // [2]
    int32_t* block_hist;   // [route_blocks * E] scratch of the counting sort
    uint32_t max_tiles;
    uint32_t max_pad_rows;
    uint32_t route_blocks;
    uint32_t tile_rows;    // rows of one tile: expert segments are padded to a multiple of it
};

size_t route_tables_bytes(uint32_t routes, uint32_t experts);
// Carves the tables out of `base` (may be NULL for sizing); returns bytes used.
size_t route_tables_carve(char* base, uint32_t routes, uint32_t experts, RouteTables* out,
                          uint32_t tile_rows = kTileM);
// Counting sort of the routes by local expert, stable in route index.
cudaError_t launch_route_sort(const int32_t* topk_ids, const float* topk_weights, uint32_t routes,
                              uint32_t top_k, uint32_t local_offset, uint32_t experts,
                              const RouteTables& rt, cudaStream_t stream);

// ---- router -----------------------------------------------------------------------
// `bias` (optional f32 [num_experts]) is added to the logits before scoring.
cudaError_t launch_router_topk(const void* logits, int logits_bf16, const float* bias,
                               int32_t* ids, float* weights, uint32_t num_tokens,
                               uint32_t num_experts, uint32_t top_k, int sigmoid_score,
                               int renormalize, float scaling, cudaStream_t stream);
qsfi_status validate_router_desc(const qscu_router_topk_desc* d);

// ---- permute / combine ----------------------------------------------------------
cudaError_t launch_gather_bf16(const __nv_bfloat16* hidden, const int32_t* route_prows,
                               uint32_t routes, uint32_t top_k, uint32_t hidden_size,
                               __nv_bfloat16* expanded, cudaStream_t stream);

// dst[prow(route), :] = src[route / top_k, :] for rows of row_bytes (a multiple of 4) bytes.
cudaError_t launch_gather_rows(const void* src, uint32_t row_bytes, const int32_t* route_prows, uint32_t routes,
                               uint32_t top_k, void* dst, cudaStream_t stream);

struct CombineParams {
    const int32_t* route_prows;   // [T*K]
    const float* topk_weights;    // [T*K]
    const __nv_bfloat16* expert_out; // [pad_rows, H]
    __nv_bfloat16* out;           // [T, H]
    uint32_t num_tokens, top_k, hidden_size;
    // optional shared expert term: out += sigmoid(x . gate_w) * shared_out
    const __nv_bfloat16* shared_out; // [T, H] or NULL
    const __nv_bfloat16* hidden;     // [T, H] for the gate logit
    const __nv_bfloat16* gate_w;     // [H]
    int round_before_shared;         // 1: round the routed sum to bf16 first (upstream chain)
    int skip_empty;                  // 1: leave rows of tokens without any local route unwritten
    // optional post-MoE neighbours fused in (hidden_size <= 2048): residual += out (bf16, in
    // place) and out = rmsnorm(residual) * norm_weight, as qsfi_fused_add_rmsnorm would do
    __nv_bfloat16* residual;         // [T, H] or NULL
    const __nv_bfloat16* norm_weight; // [H]
    float norm_eps;
};

struct EpPullParams {
    const __nv_bfloat16* peer[32];   // every rank's partial-sum buffer [num_ranks * T, H] (peer-mapped)
    const int32_t* topk_ids;         // [T, K] this rank's routing (global expert ids)
    __nv_bfloat16* out;              // [T, H]
    const __nv_bfloat16* shared_out; // optional [T, H]
    const __nv_bfloat16* hidden;     // [T, H]
    const __nv_bfloat16* gate_w;     // [H]
    uint32_t num_tokens, top_k, hidden_size, num_ranks, my_rank, experts_per_rank;
    uint32_t dbg; // measurement only (QS3_EP_FINISH_DBG): 1 read the own rank's partial sums only
};
cudaError_t launch_ep_pull_combine(const EpPullParams& p, cudaStream_t stream);
struct EpPullTokensParams {
    const uint8_t* peer[32];    // every rank's symmetric token block (peer-mapped)
    uint64_t seg_offset[4];     // byte offset of segment j inside a token block
    uint64_t seg_bytes[4];      // bytes of segment j per rank (multiple of 16)
    uint8_t* dst[4];            // local buffer of segment j: [num_ranks, seg_bytes[j]]
    uint32_t num_ranks, num_segments;
};
cudaError_t launch_ep_pull_tokens(const EpPullTokensParams& p, cudaStream_t stream);
cudaError_t launch_combine(const CombineParams& p, cudaStream_t stream);
struct EpBarrierParams {
    uint32_t* pads[32];     // pads[r]: rank r's signal pad (num_ranks words) as mapped on this device
    uint32_t num_ranks, my_rank, epoch;
    uint32_t* epoch_counter; // optional: epoch = *counter + 1, stored back by the kernel
    uint64_t limit_cycles;
    uint32_t* err;
};
cudaError_t launch_ep_barrier(const EpBarrierParams& p, cudaStream_t stream);
cudaError_t launch_ep_route_targets(const int32_t* ids, const int32_t* map, uint32_t map_len, int32_t* out,
                                    uint32_t* mask, uint32_t tokens, uint32_t top_k, uint32_t per_rank,
                                    uint32_t ranks, cudaStream_t stream);
struct EpPullRoutedParams {
    const uint8_t* peer[32];   // every rank's peer-mapped token block
    uint64_t off_codes, off_scales, off_ids, off_wts, off_mask; // byte offsets of the segments in a block
    uint8_t *dst_codes, *dst_scales, *dst_ids, *dst_wts;        // local [num_ranks * num_tokens, ...] buffers
    uint32_t num_ranks, my_rank, num_tokens, top_k;
    uint32_t code_vecs, scale_vecs; // 16-byte vectors per row of codes (<= 64) / scales (<= 32)
};
cudaError_t launch_ep_pull_routed(const EpPullRoutedParams& p, cudaStream_t stream);
cudaError_t launch_ep_rank_routes(int32_t* rows, float* weights, uint32_t tokens, uint32_t ranks,
                                  cudaStream_t stream);

// ---- GEMMs ----------------------------------------------------------------------
enum GemmEpilogue {
    EPI_STORE_BF16 = 0,   // out = bf16(alpha * acc [+ beta * out])
    EPI_STORE_F32 = 1,    // out = alpha * acc [+ beta * out] [+ bias[n]]
    EPI_SWIGLU_BF16 = 2,  // out = bf16(silu(bf16(g)) * bf16(u))
    EPI_SWIGLU_NVFP4 = 3  // out = nvfp4(silu(g) * u), packed + tiled scales
};

struct GemmProblem {
    // A operand: [a_rows, k] row-major (bf16 elements or packed e2m1 bytes), pitch in BYTES
    const void* a;
    uint64_t a_rows;
    uint64_t a_pitch_bytes;
    const uint8_t* a_scale_tiled; // NVFP4 only
    // B operand: [groups, b_rows, k]; b_rows = 2*n for gated problems
    const void* b;
    uint64_t b_pitch_bytes;
    const uint8_t* b_scale_tiled; // NVFP4 only, per group qs3_nvfp4_tiled_scale_bytes(b_rows, k)
    uint32_t groups;
    uint32_t n; // output features (gated: intermediate size)
    uint32_t k; // reduction length in elements
    int nvfp4;
    int gated;
    int epilogue;
    // tile tables (NULL: dense problem, tiles are consecutive 128-row blocks of A)
    const int32_t* tile_expert;
    const int32_t* tile_row0;
    const int32_t* tile_nrows;
    const int32_t* total_tiles;
    uint32_t max_tiles;
    uint32_t tile_rows;  // rows per tile of the tables: 128, or 32 (NVFP4 decode kernel, operands swapped)
    uint32_t est_tiles;  // expected number of tiles (sizes the splits of the decode kernel), 0: unknown
    // pair tiles of the route sort (RouteTables::pair_*), NULL: no CTA-pair kernel for this problem
    const int32_t* pair_expert;
    const int32_t* pair_row0;
    const int32_t* pair_nrows;
    const int32_t* pair_counts;
    // output
    void* out;
    uint64_t out_pitch_elems;   // elements (bytes for packed NVFP4 output)
    uint8_t* out_scale_tiled;   // EPI_SWIGLU_NVFP4
    float alpha;                // 0 means 1
    float beta;
    const float* group_scale;   // optional per-group multiplier on acc
    const float* group_scale_up; // gated: optional multiplier of the up rows (NULL: group_scale)
    const float* bias;          // optional f32 [n] (EPI_STORE_F32)
    float out_global_scale;     // EPI_SWIGLU_NVFP4: global scale of the quantised output
    // optional scratch for split-k (dense bf16 problems with f32 output, few output tiles and a long k:
    // router logits of a decode batch); NULL: never split
    float* splitk_scratch;
    size_t splitk_scratch_bytes;
};
// Chooses the tcgen05 kernel when the shape allows it and the plain CUDA-core
// kernel otherwise (tiny or unaligned shapes; bf16 only).
cudaError_t launch_gemm(const GemmProblem& p, cudaStream_t stream, const char** why_unsupported);
// Persistent 128 x 256 kernel for dense bf16 problems with more than 64 rows (gemm_dense.cu).
bool gemm_dense_bf16_supported(const GemmProblem& p);
cudaError_t launch_gemm_dense_bf16(const GemmProblem& p, cudaStream_t stream, const char** why_unsupported);
// NVFP4 GEMM on CTA pairs (256 x 256 instructions, weights cross L2 -> SM once per 256 rows; gemm_pair.cu).
bool nvfp4_pair_gemm_supported(const GemmProblem& p);
cudaError_t launch_nvfp4_pair_gemm(const GemmProblem& p, cudaStream_t stream, const char** why_unsupported);
// NVFP4 grouped GEMM for 32-row token tiles (decode batches): weights are the M side of the MMA.
cudaError_t launch_nvfp4_swap_gemm(const GemmProblem& p, cudaStream_t stream, const char** why_unsupported);
// Rows per token tile of an NVFP4 plan: 32 (decode kernel) when experts get few rows each, else 128.
uint32_t nvfp4_tile_rows(uint32_t routes, uint32_t experts, uint32_t hidden, uint32_t inter);
bool gemm_tc_supported(const GemmProblem& p);

// ---- NVFP4 ----------------------------------------------------------------------
cudaError_t launch_nvfp4_gather_quantize(const __nv_bfloat16* hidden, const int32_t* route_prows,
                                         uint32_t routes, uint32_t top_k, uint32_t hidden_size,
                                         float global_scale, uint8_t* packed, uint8_t* scale_tiled,
                                         cudaStream_t stream);
// Gather of already-quantised token rows into the padded permuted layout of sorted routing tables.
// 128-row tiles: organised by destination tile (coalesced code rows, whole scale tiles; rows past a
// tile's last row keep stale codes and get zero scales); smaller tiles: launch_nvfp4_gather_packed.
cudaError_t launch_nvfp4_gather_tiles(const uint8_t* hidden_packed, const uint8_t* hidden_scale, const RouteTables& rt,
                                      uint32_t routes, uint32_t top_k, uint32_t hidden_size, uint8_t* packed,
                                      uint8_t* scale_tiled, cudaStream_t stream, int src_scale_tiled = 0);
// `src_scale_tiled`: the source scales are tiled by token row instead of row-major.
cudaError_t launch_nvfp4_gather_packed(const uint8_t* hidden_packed, const uint8_t* hidden_scale,
                                       const int32_t* route_prows, uint32_t routes, uint32_t top_k,
                                       uint32_t hidden_size, uint8_t* packed, uint8_t* scale_tiled,
                                       cudaStream_t stream, int src_scale_tiled = 0);

// ---- FP8 (e4m3, 128 x 128 weight blocks, per-token 128-element activation groups) ----
// Rows of one token tile of the FP8 grouped GEMM for this many routes over this many experts.
uint32_t fp8_tile_rows(uint32_t routes, uint32_t experts);
// codes[prow] / scales[prow] = quantise(x[route / top_k]); route_prows NULL: dense, prow = route.
cudaError_t launch_fp8_gather_quantize(const __nv_bfloat16* x, const int32_t* route_prows, uint32_t routes,
                                       uint32_t top_k, uint32_t k, uint8_t* codes, float* scales,
                                       cudaStream_t stream);
cudaError_t launch_fp8_quantize_weight(const __nv_bfloat16* w, uint32_t experts, uint32_t rows, uint32_t k,
                                       uint8_t* codes, float* scales, cudaStream_t stream);
struct Fp8Gemm {
    const uint8_t* x;        // e4m3 [x_rows, k], rows in the padded (tile_rows) layout
    const float* x_scale;    // [x_rows, k / 128]
    uint64_t x_rows;
    const uint8_t* w;        // e4m3 [groups, gated ? 2n : n, k]
    const float* w_scale;    // [groups, ceil(rows / 128), k / 128]
    uint32_t groups, n, k;
    int gated;               // 1: out = quantise(silu(gate) * up) as e4m3 [x_rows, n] + out_scale
    const int32_t* tile_expert;
    const int32_t* tile_row0;
    const int32_t* tile_nrows;
    const int32_t* total_tiles;
    uint32_t max_tiles;
    uint32_t est_tiles;      // host-side estimate of *total_tiles, sizes the feature splits
    uint32_t tile_rows;      // 16 or 32
    void* out;               // gated: u8 [x_rows, n]; else bf16 [x_rows, n]
    float* out_scale;        // gated: f32 [x_rows, n / 128]
};
cudaError_t launch_fp8_gemm(const Fp8Gemm& g, cudaStream_t stream, const char** why_unsupported);

// ---- device helpers ---------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16)
{
    return __uint_as_float(bits16 << 16);
}
// upstream qscu.cu:253-256 / qsfi_moe.cu:461
__device__ __forceinline__ float sigmoid_fast(float v) { return 1.0f / (1.0f + __expf(-v)); }
#endif

} // namespace qs3
