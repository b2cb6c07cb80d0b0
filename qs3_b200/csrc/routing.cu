// Route permutation (histogram, scan, stable placement), token gather and the
// weighted combine. Replaces upstream count_routes / prefix_sum / fill_route_rows /
// scatter_hidden / finalize (qsfi_moe.cu:327-409,465-492).
#include "common.cuh"

#include <algorithm>
#include <cstdlib>

#include <mutex>

namespace qs3 {

namespace {

constexpr int kSortWarps = 8;              // warps per block of the counting sort
constexpr int kSortRounds = 4;              // 32-route rounds per warp
constexpr int kSortChunk = kSortWarps * kSortRounds * 32; // routes per block (1024)

__device__ __forceinline__ int local_expert(const int32_t* ids, uint32_t route, uint32_t routes,
                                            uint32_t local_offset, uint32_t experts)
{
    if (route >= routes)
        return -1;
    const int local = ids[route] - static_cast<int>(local_offset);
    return (local < 0 || local >= static_cast<int>(experts)) ? -1 : local;
}

// Per-warp histogram of the block's routes into s_hist[warp][expert] (u16: a warp
// sees at most kSortRounds * 32 routes). Each warp owns a contiguous run of routes,
// which is what makes the later placement stable.
__device__ __forceinline__ void
warp_histogram(const int32_t* ids, uint32_t routes, uint32_t local_offset, uint32_t experts,
               uint16_t* s_hist, uint32_t chunk)
{
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t i = threadIdx.x; i < kSortWarps * experts; i += blockDim.x)
        s_hist[i] = 0;
    __syncthreads();
    uint16_t* mine = s_hist + static_cast<size_t>(warp) * experts;
    const uint32_t base = chunk * kSortChunk + warp * (kSortRounds * 32);
#pragma unroll
    for (int r = 0; r < kSortRounds; ++r) {
        const int e = local_expert(ids, base + r * 32 + lane, routes, local_offset, experts);
        const uint32_t peers = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && lane == static_cast<uint32_t>(__ffs(peers) - 1))
            mine[e] += static_cast<uint16_t>(__popc(peers));
        __syncwarp();
    }
    __syncthreads();
}

__device__ __forceinline__ void route_hist_body(const int32_t* __restrict__ ids, uint32_t routes,
                                                uint32_t local_offset, uint32_t experts,
                                                int32_t* __restrict__ block_hist, uint16_t* s_hist, uint32_t chunk)
{
    warp_histogram(ids, routes, local_offset, experts, s_hist, chunk);
    for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) {
        int total = 0;
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w)
            total += s_hist[static_cast<size_t>(w) * experts + e];
        block_hist[static_cast<size_t>(chunk) * experts + e] = total;
    }
}

__global__ void __launch_bounds__(kSortWarps * 32)
route_hist_kernel(const int32_t* __restrict__ ids, uint32_t routes, uint32_t local_offset,
                  uint32_t experts, int32_t* __restrict__ block_hist)
{
    extern __shared__ uint16_t s_hist[];
    route_hist_body(ids, routes, local_offset, experts, block_hist, s_hist, blockIdx.x);
}

// Single block: per expert, exclusive scan of the block histograms (column scan),
// then exclusive scans over experts of the counts, of the counts padded to the
// tile height, and of the tile counts; finally the tile table.
__device__ __forceinline__ void route_scan_body(int32_t* __restrict__ block_hist, uint32_t num_blocks,
                                                uint32_t experts, const RouteTables& rt)
{
    constexpr int kScans = 5; // counts, padded counts, tiles, full pair tiles, single tiles
    __shared__ int s_warp[kScans][32];
    __shared__ int s_carry[kScans];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < kScans)
        s_carry[threadIdx.x] = 0;
    __syncthreads();
    for (uint32_t e0 = 0; e0 < experts; e0 += blockDim.x) {
        const uint32_t e = e0 + threadIdx.x;
        int count = 0;
        if (e < experts) {
            // loads are issued in independent batches so that their latencies overlap
            constexpr uint32_t kBatch = 16;
            for (uint32_t b0 = 0; b0 < num_blocks; b0 += kBatch) {
                int v[kBatch];
#pragma unroll
                for (uint32_t j = 0; j < kBatch; ++j)
                    v[j] = b0 + j < num_blocks
                        ? block_hist[static_cast<size_t>(b0 + j) * experts + e]
                        : 0;
#pragma unroll
                for (uint32_t j = 0; j < kBatch; ++j) {
                    if (b0 + j < num_blocks)
                        block_hist[static_cast<size_t>(b0 + j) * experts + e] = count;
                    count += v[j];
                }
            }
            rt.counts[e] = count;
        }
        const int tile_rows = static_cast<int>(rt.tile_rows);
        const int tiles = (count + tile_rows - 1) / tile_rows;
        const bool pairing = rt.pair_expert != nullptr;
        int v[kScans] = { count, tiles * tile_rows, tiles, pairing ? tiles >> 1 : 0, pairing ? tiles & 1 : 0 };
        int incl[kScans];
#pragma unroll
        for (int j = 0; j < kScans; ++j) {
            int x = v[j];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, x, o);
                if (lane >= static_cast<uint32_t>(o))
                    x += y;
            }
            incl[j] = x;
            if (lane == 31)
                s_warp[j][warp] = x;
            if (threadIdx.x < 32 && threadIdx.x >= blockDim.x / 32)
                s_warp[j][threadIdx.x] = 0; // slots of warps this block does not have
        }
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int j = 0; j < kScans; ++j) {
                int x = s_warp[j][lane];
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int y = __shfl_up_sync(0xffffffffu, x, o);
                    if (lane >= static_cast<uint32_t>(o))
                        x += y;
                }
                s_warp[j][lane] = x; // inclusive over warps
            }
        }
        __syncthreads();
        int excl[kScans];
#pragma unroll
        for (int j = 0; j < kScans; ++j)
            excl[j] = s_carry[j] + (warp > 0 ? s_warp[j][warp - 1] : 0) + incl[j] - v[j];
        if (e < experts) {
            rt.indptr[e] = excl[0];
            rt.pad_indptr[e] = excl[1];
            for (int m = 0; m < tiles; ++m) {
                rt.tile_expert[excl[2] + m] = static_cast<int32_t>(e);
                rt.tile_row0[excl[2] + m] = excl[1] + m * tile_rows;
                rt.tile_nrows[excl[2] + m] = min(tile_rows, count - m * tile_rows);
            }
            if (pairing) {
                for (int m = 0; m < (tiles >> 1); ++m) {
                    rt.pair_expert[excl[3] + m] = static_cast<int32_t>(e);
                    rt.pair_row0[excl[3] + m] = excl[1] + m * 2 * tile_rows;
                    rt.pair_nrows[excl[3] + m] = min(2 * tile_rows, count - m * 2 * tile_rows);
                }
                if (tiles & 1) {
                    const int at = static_cast<int>(rt.max_tiles) - 1 - excl[4];
                    rt.pair_expert[at] = static_cast<int32_t>(e);
                    rt.pair_row0[at] = excl[1] + (tiles - 1) * tile_rows;
                    rt.pair_nrows[at] = count - (tiles - 1) * tile_rows;
                }
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
#pragma unroll
            for (int j = 0; j < kScans; ++j)
                s_carry[j] += s_warp[j][31];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        rt.indptr[experts] = s_carry[0];
        rt.pad_indptr[experts] = s_carry[1];
        *rt.total_tiles = s_carry[2];
        if (rt.pair_counts != nullptr) {
            rt.pair_counts[0] = s_carry[3];
            rt.pair_counts[1] = s_carry[4];
        }
    }
}

__global__ void __launch_bounds__(1024)
route_scan_kernel(int32_t* __restrict__ block_hist, uint32_t num_blocks, uint32_t experts,
                  RouteTables rt)
{
    route_scan_body(block_hist, num_blocks, experts, rt);
}

// Placement: row of a route = segment start + routes of the same expert in earlier
// blocks + in earlier warps of this block + earlier in this warp. Stable in route
// index, so the permutation is reproducible (upstream's is atomics-ordered).
// `s_hist` holds the per-warp histograms of this block (warp_histogram).
__device__ __forceinline__ void route_place_body(const int32_t* __restrict__ ids,
                                                 const float* __restrict__ weights, uint32_t routes,
                                                 uint32_t top_k, uint32_t local_offset, uint32_t experts,
                                                 const RouteTables& rt, uint16_t* s_hist, uint32_t chunk)
{
    // exclusive prefix over the warps of the block, per expert
    for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) {
        int run = 0;
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) {
            const size_t i = static_cast<size_t>(w) * experts + e;
            const int v = s_hist[i];
            s_hist[i] = static_cast<uint16_t>(run);
            run += v;
        }
    }
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint16_t* mine = s_hist + static_cast<size_t>(warp) * experts;
    const uint32_t base = chunk * kSortChunk + warp * (kSortRounds * 32);
    const int32_t* block_off = rt.block_hist + static_cast<size_t>(chunk) * experts;
#pragma unroll
    for (int r = 0; r < kSortRounds; ++r) {
        const uint32_t route = base + r * 32 + lane;
        const int e = local_expert(ids, route, routes, local_offset, experts);
        const uint32_t peers = __match_any_sync(0xffffffffu, e);
        int in_block = 0;
        if (e >= 0)
            in_block = mine[e] + __popc(peers & ((1u << lane) - 1u));
        __syncwarp();
        if (e >= 0 && lane == static_cast<uint32_t>(__ffs(peers) - 1))
            mine[e] += static_cast<uint16_t>(__popc(peers));
        __syncwarp();
        if (route < routes) {
            if (e >= 0) {
                const int off = block_off[e] + in_block;
                const int row = rt.indptr[e] + off;
                rt.route_rows[route] = row;
                rt.route_prows[route] = rt.pad_indptr[e] + off;
                rt.row_tokens[row] = static_cast<int32_t>(route / top_k);
                rt.row_scales[row] = weights[route];
            } else {
                rt.route_rows[route] = -1;
                rt.route_prows[route] = -1;
            }
        }
    }
}

__global__ void __launch_bounds__(kSortWarps * 32)
route_place_kernel(const int32_t* __restrict__ ids, const float* __restrict__ weights,
                   uint32_t routes, uint32_t top_k, uint32_t local_offset, uint32_t experts,
                   RouteTables rt)
{
    extern __shared__ uint16_t s_hist[];
    warp_histogram(ids, routes, local_offset, experts, s_hist, blockIdx.x);
    route_place_body(ids, weights, routes, top_k, local_offset, experts, rt, s_hist, blockIdx.x);
}

// All three steps in one block when the routes fit a few chunks (decode batches): the same
// arithmetic as the three kernels, chunk after chunk, without two launch boundaries. The per-warp
// histograms of every chunk stay in shared memory between the first and the last step.
constexpr uint32_t kSmallSortChunks = 4;
__global__ void __launch_bounds__(kSortWarps * 32)
route_sort_small_kernel(const int32_t* __restrict__ ids, const float* __restrict__ weights,
                        uint32_t routes, uint32_t top_k, uint32_t local_offset, uint32_t experts,
                        RouteTables rt)
{
    extern __shared__ uint16_t s_hist[];
    const size_t per_chunk = static_cast<size_t>(kSortWarps) * experts;
    for (uint32_t c = 0; c < rt.route_blocks; ++c)
        route_hist_body(ids, routes, local_offset, experts, rt.block_hist, s_hist + c * per_chunk, c);
    __syncthreads(); // block_hist (global) is read back by this block
    route_scan_body(rt.block_hist, rt.route_blocks, experts, rt);
    __syncthreads(); // indptr / pad_indptr and the scanned block_hist (global) are read back by this block
    for (uint32_t c = 0; c < rt.route_blocks; ++c)
        route_place_body(ids, weights, routes, top_k, local_offset, experts, rt, s_hist + c * per_chunk, c);
}

// expanded[prow, :] = hidden[route / top_k, :]; one warp per route, 16-byte copies.
__global__ void __launch_bounds__(256)
gather_bf16_kernel(const uint4* __restrict__ hidden, const int32_t* __restrict__ route_prows,
                   uint32_t routes, uint32_t top_k, uint32_t vec_per_row,
                   uint4* __restrict__ expanded)
{
    const uint32_t route = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (route >= routes)
        return;
    const int prow = route_prows[route];
    if (prow < 0)
        return;
    const uint4* src = hidden + static_cast<size_t>(route / top_k) * vec_per_row;
    uint4* dst = expanded + static_cast<size_t>(prow) * vec_per_row;
    for (uint32_t i = threadIdx.x & 31; i < vec_per_row; i += 32)
        dst[i] = src[i];
}

// Same gather for rows whose length is only a multiple of 4 bytes.
__global__ void __launch_bounds__(256)
gather_words_kernel(const uint32_t* __restrict__ src, const int32_t* __restrict__ route_prows,
                    uint32_t routes, uint32_t top_k, uint32_t words_per_row, uint32_t* __restrict__ dst)
{
    const uint32_t route = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (route >= routes)
        return;
    const int prow = route_prows[route];
    if (prow < 0)
        return;
    const uint32_t* s = src + static_cast<size_t>(route / top_k) * words_per_row;
    uint32_t* d = dst + static_cast<size_t>(prow) * words_per_row;
    for (uint32_t i = threadIdx.x & 31; i < words_per_row; i += 32)
        d[i] = s[i];
}

// out[t, :] = bf16(sum_k w[t,k] * f32(Y2[prow(t,k), :])) (+ shared-expert term).
// Four tokens per block, 64 threads per token; a thread owns two 8-element chunks of the row
// per step and issues the loads of up to four routes for both chunks together (eight 16-byte
// loads in flight), so that tokens with one or two local routes (expert parallelism) still
// keep the memory system busy. k ascending and f32 accumulation as upstream finalize_kernel
// (qsfi_moe.cu:465-492).
constexpr uint32_t kCombineTokens = 4;
constexpr uint32_t kCombineGroup = 64;

__device__ __forceinline__ void accumulate_row(float* acc, const uint4& v, float w)
{
    const uint32_t vs[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        acc[2 * j] += w * bf16_bits_to_f32(vs[j] & 0xffffu);
        acc[2 * j + 1] += w * bf16_bits_to_f32(vs[j] >> 16);
    }
}

__global__ void __launch_bounds__(kCombineTokens* kCombineGroup, 4) combine_kernel(CombineParams p)
{
    __shared__ int s_row[kCombineTokens][32];
    __shared__ float s_w[kCombineTokens][32];
    __shared__ float s_dot[kCombineTokens][kCombineGroup / 32];
    __shared__ int s_any[kCombineTokens];
    const uint32_t group = threadIdx.x / kCombineGroup, gl = threadIdx.x % kCombineGroup;
    const uint32_t token = blockIdx.x * kCombineTokens + group;
    const bool live = token < p.num_tokens;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t vec_per_row = p.hidden_size / 8;

    if (gl < 32) {
        // the token's routes that have a row here, compacted in ascending k
        int row = -1;
        float wgt = 0.0f;
        if (live && gl < p.top_k) {
            row = p.route_prows[static_cast<size_t>(token) * p.top_k + gl];
            wgt = p.topk_weights[static_cast<size_t>(token) * p.top_k + gl];
        }
        const uint32_t valid = __ballot_sync(0xffffffffu, row >= 0);
        if (row >= 0) {
            const uint32_t slot = __popc(valid & ((1u << gl) - 1u));
            s_row[group][slot] = row;
            s_w[group][slot] = wgt;
        }
        if (gl == 0)
            s_any[group] = __popc(valid);
    }
    float dot = 0.0f;
    if (p.shared_out != nullptr) {
        // gate logit x . w_gate in f32 (upstream computes it as an N = 1 GEMM,
        // src/model.rs:2218-2226)
        if (live) {
            const uint4* x = reinterpret_cast<const uint4*>(p.hidden) + static_cast<size_t>(token) * vec_per_row;
            const uint4* w = reinterpret_cast<const uint4*>(p.gate_w);
            for (uint32_t i = gl; i < vec_per_row; i += kCombineGroup) {
                const uint4 xv = x[i], wv = w[i];
                const uint32_t xs[4] = { xv.x, xv.y, xv.z, xv.w };
                const uint32_t ws[4] = { wv.x, wv.y, wv.z, wv.w };
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dot += bf16_bits_to_f32(xs[j] & 0xffffu) * bf16_bits_to_f32(ws[j] & 0xffffu);
                    dot += bf16_bits_to_f32(xs[j] >> 16) * bf16_bits_to_f32(ws[j] >> 16);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0)
            s_dot[group][gl / 32] = dot;
    }
    __syncthreads();
    if (!live || (p.skip_empty && !s_any[group]))
        return; // no local route: the row stays unwritten and is never read
    float gate = 0.0f;
    if (p.shared_out != nullptr) {
        dot = 0.0f;
#pragma unroll
        for (uint32_t w = 0; w < kCombineGroup / 32; ++w) // fixed order: the same sum in every thread
            dot += s_dot[group][w];
        gate = sigmoid_fast(dot);
    }

    const uint4* y2 = reinterpret_cast<const uint4*>(p.expert_out);
    uint4* out = reinterpret_cast<uint4*>(p.out) + static_cast<size_t>(token) * vec_per_row;
    const uint32_t n_valid = static_cast<uint32_t>(s_any[group]);
    for (uint32_t i0 = gl; i0 < vec_per_row; i0 += 2 * kCombineGroup) {
        const uint32_t i1 = i0 + kCombineGroup;
        const bool two = i1 < vec_per_row;
        float acc0[8], acc1[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            acc0[j] = acc1[j] = 0.0f;
        for (uint32_t k0 = 0; k0 < n_valid; k0 += 4) {
            uint4 v0[4], v1[4];
            float w[4];
            int row[4];
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q) {
                row[q] = k0 + q < n_valid ? s_row[group][k0 + q] : -1;
                w[q] = row[q] >= 0 ? s_w[group][k0 + q] : 0.0f;
                const uint4* src = y2 + static_cast<size_t>(row[q] >= 0 ? row[q] : 0) * vec_per_row;
                v0[q] = row[q] >= 0 ? src[i0] : make_uint4(0, 0, 0, 0);
                v1[q] = (row[q] >= 0 && two) ? src[i1] : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q) {
                if (row[q] < 0)
                    continue; // a skipped route adds nothing (not even a signed zero)
                accumulate_row(acc0, v0[q], w[q]);
                accumulate_row(acc1, v1[q], w[q]);
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float* acc = h == 0 ? acc0 : acc1;
            const uint32_t i = h == 0 ? i0 : i1;
            if (h == 1 && !two)
                break;
            if (p.shared_out != nullptr) {
                const uint4 sv
                    = reinterpret_cast<const uint4*>(p.shared_out)[static_cast<size_t>(token) * vec_per_row + i];
                const uint32_t ss[4] = { sv.x, sv.y, sv.z, sv.w };
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float a0 = acc[2 * j], a1 = acc[2 * j + 1];
                    if (p.round_before_shared) { // upstream rounds the routed sum to bf16 first
                        a0 = __bfloat162float(__float2bfloat16(a0));
                        a1 = __bfloat162float(__float2bfloat16(a1));
                    }
                    acc[2 * j] = a0 + gate * bf16_bits_to_f32(ss[j] & 0xffffu);
                    acc[2 * j + 1] = a1 + gate * bf16_bits_to_f32(ss[j] >> 16);
                }
            }
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 r = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                o[j] = *reinterpret_cast<const uint32_t*>(&r);
            }
            out[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// The combine above followed by the block's post-MoE neighbours in the same pass:
//   x        = bf16(sum_k w_k * Y2[row_k] (+ shared term))        (what combine_kernel stores)
//   residual = bf16(f32(x) + f32(residual))                       (in place)
//   out      = bf16((f32(x) + f32(residual)) * rsqrt(mean(.^2) + eps) * norm_weight)
// i.e. qsfi_fused_add_rmsnorm applied to the MoE output without the round trip of [T, H]
// through HBM. A thread keeps its four chunks of the row in registers across the row-wide
// reduction, so rows are limited to 4 * 64 * 8 = 2048 elements.
__global__ void __launch_bounds__(kCombineTokens* kCombineGroup, 2) combine_norm_kernel(CombineParams p)
{
    __shared__ int s_row[kCombineTokens][32];
    __shared__ float s_w[kCombineTokens][32];
    __shared__ float s_dot[kCombineTokens][kCombineGroup / 32];
    __shared__ float s_sq[kCombineTokens][kCombineGroup / 32];
    __shared__ int s_any[kCombineTokens];
    const uint32_t group = threadIdx.x / kCombineGroup, gl = threadIdx.x % kCombineGroup;
    const uint32_t token = blockIdx.x * kCombineTokens + group;
    const bool live = token < p.num_tokens;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t vec_per_row = p.hidden_size / 8;

    if (gl < 32) {
        int row = -1;
        float wgt = 0.0f;
        if (live && gl < p.top_k) {
            row = p.route_prows[static_cast<size_t>(token) * p.top_k + gl];
            wgt = p.topk_weights[static_cast<size_t>(token) * p.top_k + gl];
        }
        const uint32_t valid = __ballot_sync(0xffffffffu, row >= 0);
        if (row >= 0) {
            const uint32_t slot = __popc(valid & ((1u << gl) - 1u));
            s_row[group][slot] = row;
            s_w[group][slot] = wgt;
        }
        if (gl == 0)
            s_any[group] = __popc(valid);
    }
    float dot = 0.0f;
    if (p.shared_out != nullptr) {
        if (live) {
            const uint4* x = reinterpret_cast<const uint4*>(p.hidden) + static_cast<size_t>(token) * vec_per_row;
            const uint4* w = reinterpret_cast<const uint4*>(p.gate_w);
            for (uint32_t i = gl; i < vec_per_row; i += kCombineGroup) {
                const uint4 xv = x[i], wv = w[i];
                const uint32_t xs[4] = { xv.x, xv.y, xv.z, xv.w };
                const uint32_t ws[4] = { wv.x, wv.y, wv.z, wv.w };
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dot += bf16_bits_to_f32(xs[j] & 0xffffu) * bf16_bits_to_f32(ws[j] & 0xffffu);
                    dot += bf16_bits_to_f32(xs[j] >> 16) * bf16_bits_to_f32(ws[j] >> 16);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0)
            s_dot[group][gl / 32] = dot;
    }
    __syncthreads();
    float gate = 0.0f;
    if (p.shared_out != nullptr) {
        dot = 0.0f;
#pragma unroll
        for (uint32_t w = 0; w < kCombineGroup / 32; ++w)
            dot += s_dot[group][w];
        gate = sigmoid_fast(dot);
    }

    const uint4* y2 = reinterpret_cast<const uint4*>(p.expert_out);
    const uint32_t n_valid = live ? static_cast<uint32_t>(s_any[group]) : 0u;
    uint4* res = reinterpret_cast<uint4*>(p.residual) + static_cast<size_t>(live ? token : 0) * vec_per_row;
    float vals[4][8]; // chunks gl, gl + 64, gl + 128, gl + 192 of the row
    float sum_sq = 0.0f;
#pragma unroll
    for (uint32_t step = 0; step < 2; ++step) {
        const uint32_t i0 = gl + step * 2 * kCombineGroup, i1 = i0 + kCombineGroup;
        const bool one = live && i0 < vec_per_row, two = live && i1 < vec_per_row;
        float* acc0 = vals[2 * step];
        float* acc1 = vals[2 * step + 1];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            acc0[j] = acc1[j] = 0.0f;
        for (uint32_t k0 = 0; k0 < n_valid; k0 += 4) {
            uint4 v0[4], v1[4];
            float w[4];
            int row[4];
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q) {
                row[q] = k0 + q < n_valid ? s_row[group][k0 + q] : -1;
                w[q] = row[q] >= 0 ? s_w[group][k0 + q] : 0.0f;
                const uint4* src = y2 + static_cast<size_t>(row[q] >= 0 ? row[q] : 0) * vec_per_row;
                v0[q] = (row[q] >= 0 && one) ? src[i0] : make_uint4(0, 0, 0, 0);
                v1[q] = (row[q] >= 0 && two) ? src[i1] : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q) {
                if (row[q] < 0)
                    continue;
                accumulate_row(acc0, v0[q], w[q]);
                accumulate_row(acc1, v1[q], w[q]);
            }
        }
#pragma unroll
        for (int hsel = 0; hsel < 2; ++hsel) {
            float* acc = hsel == 0 ? acc0 : acc1;
            const uint32_t i = hsel == 0 ? i0 : i1;
            if (!(hsel == 0 ? one : two))
                continue;
            if (p.shared_out != nullptr) {
                const uint4 sv
                    = reinterpret_cast<const uint4*>(p.shared_out)[static_cast<size_t>(token) * vec_per_row + i];
                const uint32_t ss[4] = { sv.x, sv.y, sv.z, sv.w };
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float a0 = acc[2 * j], a1 = acc[2 * j + 1];
                    if (p.round_before_shared) {
                        a0 = __bfloat162float(__float2bfloat16(a0));
                        a1 = __bfloat162float(__float2bfloat16(a1));
                    }
                    acc[2 * j] = a0 + gate * bf16_bits_to_f32(ss[j] & 0xffffu);
                    acc[2 * j + 1] = a1 + gate * bf16_bits_to_f32(ss[j] >> 16);
                }
            }
            const uint4 rv = res[i];
            const uint32_t rs[4] = { rv.x, rv.y, rv.z, rv.w };
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // the MoE output as the unfused path would have stored it, plus the residual
                const float x0 = __bfloat162float(__float2bfloat16(acc[2 * j]));
                const float x1 = __bfloat162float(__float2bfloat16(acc[2 * j + 1]));
                acc[2 * j] = x0 + bf16_bits_to_f32(rs[j] & 0xffffu);
                acc[2 * j + 1] = x1 + bf16_bits_to_f32(rs[j] >> 16);
                sum_sq += acc[2 * j] * acc[2 * j] + acc[2 * j + 1] * acc[2 * j + 1];
                const __nv_bfloat162 r2 = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                o[j] = *reinterpret_cast<const uint32_t*>(&r2);
            }
            res[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        sum_sq += __shfl_xor_sync(0xffffffffu, sum_sq, o);
    if (lane == 0)
        s_sq[group][gl / 32] = sum_sq;
    __syncthreads();
    if (!live)
        return;
    float total = 0.0f;
#pragma unroll
    for (uint32_t w = 0; w < kCombineGroup / 32; ++w)
        total += s_sq[group][w];
    const float inv_rms = 1.0f / sqrtf(total / static_cast<float>(p.hidden_size) + p.norm_eps);
    uint4* out = reinterpret_cast<uint4*>(p.out) + static_cast<size_t>(token) * vec_per_row;
    const uint4* nw = reinterpret_cast<const uint4*>(p.norm_weight);
#pragma unroll
    for (uint32_t c = 0; c < 4; ++c) {
        const uint32_t i = gl + c * kCombineGroup;
        if (i >= vec_per_row)
            continue;
        const uint4 wv = nw[i];
        const uint32_t ws[4] = { wv.x, wv.y, wv.z, wv.w };
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 r2
                = __floats2bfloat162_rn(vals[c][2 * j] * inv_rms * bf16_bits_to_f32(ws[j] & 0xffffu),
                                        vals[c][2 * j + 1] * inv_rms * bf16_bits_to_f32(ws[j] >> 16));
            o[j] = *reinterpret_cast<const uint32_t*>(&r2);
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// rows[t * ranks + r] = r * tokens + t, weights = 1: lets the combine kernel sum the
// per-rank partial rows of one token in ascending rank order.
__global__ void ep_rank_routes_kernel(int32_t* rows, float* weights, uint32_t tokens, uint32_t ranks)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= tokens * ranks)
        return;
    rows[i] = static_cast<int32_t>((i % ranks) * tokens + i / ranks);
    weights[i] = 1.0f;
}

// Per token: dispatch ids out[t, k] = map[ids[t, k]] (ids outside the map stay -1; without a map the
// ids themselves are the dispatch ids) and mask[t] = the set of ranks the token has a route to (bit r:
// some dispatch id lies in rank r's `per_rank` expert slots). The map turns the router's expert ids
// into the expert SLOTS of a placement in which every rank holds its own experts and replicas of hot ones.
__global__ void ep_route_targets_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ map,
                                        uint32_t map_len, int32_t* __restrict__ out, uint32_t* __restrict__ mask,
                                        uint32_t tokens, uint32_t top_k, uint32_t per_rank, uint32_t ranks)
{
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens)
        return;
    uint32_t m = 0;
    for (uint32_t k = 0; k < top_k; ++k) {
        int32_t id = ids[static_cast<size_t>(t) * top_k + k];
        if (map != nullptr) {
            id = (id >= 0 && static_cast<uint32_t>(id) < map_len) ? map[id] : -1;
            out[static_cast<size_t>(t) * top_k + k] = id;
        }
        if (id >= 0 && static_cast<uint32_t>(id) / per_rank < ranks)
            m |= 1u << (static_cast<uint32_t>(id) / per_rank);
    }
    if (mask != nullptr)
        mask[t] = m;
}

// Dispatch that pulls only what this rank needs: for every token of every rank, its dispatch ids
// and weights always (the route sort needs them to see that a row is not local), its NVFP4 codes and
// scales only when the token's rank mask says it has a route to an expert slot of this rank. A warp
// takes eight consecutive tokens of one peer: eight lanes fetch the masks, then the warp issues
// the loads of all wanted rows before storing any of them, so that the NVLink round trips overlap.
// Rows that are not pulled keep whatever an earlier step left there; nothing reads them, because
// none of their (fresh) ids is local. Plain peer loads; no load of this kernel is multicast.
__global__ void __launch_bounds__(256) ep_pull_routed_kernel(EpPullRoutedParams p)
{
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t groups_per_rank = (p.num_tokens + 7) / 8;
    const uint32_t group = blockIdx.x * 8 + warp;
    if (group >= groups_per_rank * p.num_ranks)
        return;
    const uint32_t r = group / groups_per_rank;
    const uint32_t t0 = (group % groups_per_rank) * 8;
    const uint8_t* peer = p.peer[r];
    const uint32_t nrows = min(8u, p.num_tokens - t0);
    uint32_t my_mask = 0;
    if (lane < nrows)
        my_mask = reinterpret_cast<const uint32_t*>(peer + p.off_mask)[t0 + lane];
    // ids and weights of the eight tokens: 8 * top_k words each, contiguous in the peer's block
    const uint32_t words = nrows * p.top_k;
    const uint32_t* ids_src = reinterpret_cast<const uint32_t*>(peer + p.off_ids) + static_cast<size_t>(t0) * p.top_k;
    const uint32_t* wts_src = reinterpret_cast<const uint32_t*>(peer + p.off_wts) + static_cast<size_t>(t0) * p.top_k;
    const size_t row0 = static_cast<size_t>(r) * p.num_tokens + t0;
    uint32_t* ids_dst = reinterpret_cast<uint32_t*>(p.dst_ids) + row0 * p.top_k;
    uint32_t* wts_dst = reinterpret_cast<uint32_t*>(p.dst_wts) + row0 * p.top_k;
    uint32_t iv[4], wv[4];
#pragma unroll
    for (uint32_t q = 0; q < 4; ++q) {
        const uint32_t i = lane + 32 * q;
        iv[q] = i < words ? ids_src[i] : 0;
        wv[q] = i < words ? wts_src[i] : 0;
    }
    uint32_t wanted = 0; // bit i: row t0 + i goes to this rank
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i)
        wanted |= ((__shfl_sync(0xffffffffu, my_mask, i) >> p.my_rank) & 1u) << i;
    // codes: code_vecs 16-byte vectors per row (<= 64 per lane pair of loads), scales: scale_vecs (<= 32)
    const uint4* codes = reinterpret_cast<const uint4*>(peer + p.off_codes);
    const uint4* scales = reinterpret_cast<const uint4*>(peer + p.off_scales);
    uint4* codes_dst = reinterpret_cast<uint4*>(p.dst_codes);
    uint4* scales_dst = reinterpret_cast<uint4*>(p.dst_scales);
    for (uint32_t i0 = 0; i0 < 8; i0 += 4) {
        uint4 c[4][2], sc[4];
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t i = i0 + j;
            const bool on = (wanted >> i) & 1u;
            const size_t src_row = t0 + i;
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h)
                if (on && lane + 32 * h < p.code_vecs)
                    c[j][h] = codes[src_row * p.code_vecs + lane + 32 * h];
            if (on && lane < p.scale_vecs)
                sc[j] = scales[src_row * p.scale_vecs + lane];
        }
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t i = i0 + j;
            if (!((wanted >> i) & 1u))
                continue;
            const size_t dst_row = row0 + i;
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h)
                if (lane + 32 * h < p.code_vecs)
                    codes_dst[dst_row * p.code_vecs + lane + 32 * h] = c[j][h];
            if (lane < p.scale_vecs)
                scales_dst[dst_row * p.scale_vecs + lane] = sc[j];
        }
    }
#pragma unroll
    for (uint32_t q = 0; q < 4; ++q) {
        const uint32_t i = lane + 32 * q;
        if (i < words) {
            ids_dst[i] = iv[q];
            wts_dst[i] = wv[q];
        }
    }
}

template <typename T> T* carve(char* base, size_t& offset, size_t count)
{
    offset = align_up(offset, kWorkspaceAlign);
    T* p = base != nullptr ? reinterpret_cast<T*>(base + offset) : nullptr;
    offset += count * sizeof(T);
    return p;
}

// Expert-parallel combine that PULLS: out[t] = bf16(sum over ranks r, ascending, of
// f32(partial_r[my_rank * T + t]) + sigmoid(x . w_gate) * shared[t]), where partial_r is
// rank r's partial-sum buffer read in place over NVLink (plain peer loads). A rank is
// read only when one of the token's routes targets one of its experts, so pairs
// (token, rank) without a route cost no traffic. Same summation order and roundings as
// exchanging the partial sums first and then running combine_kernel on the copies.
// Four tokens per block, 64 threads (two warps) per token: the kernel is bound by the latency of its
// dependent loads (ids -> which ranks -> peer rows over NVLink), so what matters is how many tokens
// are in flight per SM; with a block per token 4096 tokens took 3.5 waves of ~8 us.
constexpr uint32_t kEpTokensPerBlock = 4;

__global__ void __launch_bounds__(64 * kEpTokensPerBlock, 3) ep_pull_combine_kernel(EpPullParams p)
{
    __shared__ uint32_t s_active[kEpTokensPerBlock];
    __shared__ float s_dot[kEpTokensPerBlock][2];
    const uint32_t slot = threadIdx.x >> 6;           // token of the block
    const uint32_t tid = threadIdx.x & 63;            // thread of the token
    const uint32_t lane = threadIdx.x & 31, half = tid >> 5;
    const uint32_t token = blockIdx.x * kEpTokensPerBlock + slot;
    const bool live = token < p.num_tokens;
    const uint32_t vec_per_row = p.hidden_size / 8;

    // which ranks hold a partial sum for this token
    if (live && half == 0) {
        uint32_t mine = 0;
        if (lane < p.top_k) {
            const int id = p.topk_ids[static_cast<size_t>(token) * p.top_k + lane];
            if (id >= 0 && static_cast<uint32_t>(id) / p.experts_per_rank < p.num_ranks)
                mine = 1u << (static_cast<uint32_t>(id) / p.experts_per_rank);
        }
        const uint32_t any = __reduce_or_sync(0xffffffffu, mine);
        if (lane == 0)
            s_active[slot] = any;
    }
    float dot = 0.0f;
    if (live && p.shared_out != nullptr) {
        // gate logit: the row's loads are issued together (four chunks per thread and pass)
        const uint4* x = reinterpret_cast<const uint4*>(p.hidden) + static_cast<size_t>(token) * vec_per_row;
        const uint4* w = reinterpret_cast<const uint4*>(p.gate_w);
        for (uint32_t i0 = tid; i0 < vec_per_row; i0 += 256) {
            uint4 xv[4], wv[4];
#pragma unroll
            for (uint32_t c = 0; c < 4; ++c) {
                const uint32_t i = i0 + 64 * c;
                xv[c] = i < vec_per_row ? x[i] : make_uint4(0, 0, 0, 0);
                wv[c] = i < vec_per_row ? w[i] : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (uint32_t c = 0; c < 4; ++c) {
                const uint32_t xs[4] = { xv[c].x, xv[c].y, xv[c].z, xv[c].w };
                const uint32_t ws[4] = { wv[c].x, wv[c].y, wv[c].z, wv[c].w };
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    dot += bf16_bits_to_f32(xs[j] & 0xffffu) * bf16_bits_to_f32(ws[j] & 0xffffu);
                    dot += bf16_bits_to_f32(xs[j] >> 16) * bf16_bits_to_f32(ws[j] >> 16);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0)
            s_dot[slot][half] = dot;
    }
    __syncthreads();
    if (!live)
        return;
    const uint32_t active = (p.dbg & 1u) ? (s_active[slot] & (1u << p.my_rank)) : s_active[slot];
    float gate = 0.0f;
    if (p.shared_out != nullptr)
        gate = sigmoid_fast(s_dot[slot][0] + s_dot[slot][1]);

    const size_t row = static_cast<size_t>(p.my_rank) * p.num_tokens + token;
    uint4* out = reinterpret_cast<uint4*>(p.out) + static_cast<size_t>(token) * vec_per_row;
    // A thread owns up to four 16-byte chunks of the row (hidden <= 2048) and keeps the loads of all of
    // them, for two ranks at a time, in flight together: what bounds this kernel is the latency of the
    // peer loads, so the number of dependent rounds (ranks / 2), not the bytes, sets its time. Ranks are
    // added in ascending order.
    constexpr uint32_t kChunks = 4;
    for (uint32_t i0 = tid; i0 < vec_per_row; i0 += 64 * kChunks) {
        float acc[kChunks][8];
#pragma unroll
        for (uint32_t c = 0; c < kChunks; ++c)
#pragma unroll
            for (int j = 0; j < 8; ++j)
                acc[c][j] = 0.0f;
        // the shared expert's rows travel with the first round of partial sums
        uint4 sh[kChunks];
#pragma unroll
        for (uint32_t c = 0; c < kChunks; ++c) {
            const uint32_t i = i0 + 64 * c;
            sh[c] = (p.shared_out != nullptr && i < vec_per_row)
                ? reinterpret_cast<const uint4*>(p.shared_out)[static_cast<size_t>(token) * vec_per_row + i]
                : make_uint4(0, 0, 0, 0);
        }
        uint32_t todo = active & (p.num_ranks >= 32 ? 0xffffffffu : (1u << p.num_ranks) - 1u);
        while (todo != 0) {
            const uint32_t ra = static_cast<uint32_t>(__ffs(static_cast<int>(todo))) - 1u;
            todo &= todo - 1u;
            const bool two = todo != 0;
            const uint32_t rb = two ? static_cast<uint32_t>(__ffs(static_cast<int>(todo))) - 1u : ra;
            todo &= todo - 1u; // no-op on zero
            const uint4* pa = reinterpret_cast<const uint4*>(p.peer[ra]) + row * vec_per_row;
            const uint4* pb = reinterpret_cast<const uint4*>(p.peer[rb]) + row * vec_per_row;
            uint4 va[kChunks], vb[kChunks];
#pragma unroll
            for (uint32_t c = 0; c < kChunks; ++c) {
                const uint32_t i = i0 + 64 * c;
                va[c] = i < vec_per_row ? pa[i] : make_uint4(0, 0, 0, 0);
                vb[c] = (two && i < vec_per_row) ? pb[i] : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (uint32_t c = 0; c < kChunks; ++c) {
                const uint32_t as[4] = { va[c].x, va[c].y, va[c].z, va[c].w };
                const uint32_t bs[4] = { vb[c].x, vb[c].y, vb[c].z, vb[c].w };
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[c][2 * j] += bf16_bits_to_f32(as[j] & 0xffffu);
                    acc[c][2 * j + 1] += bf16_bits_to_f32(as[j] >> 16);
                }
                if (two) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[c][2 * j] += bf16_bits_to_f32(bs[j] & 0xffffu);
                        acc[c][2 * j + 1] += bf16_bits_to_f32(bs[j] >> 16);
                    }
                }
            }
        }
#pragma unroll
        for (uint32_t c = 0; c < kChunks; ++c) {
            const uint32_t i = i0 + 64 * c;
            if (i >= vec_per_row)
                break;
            if (p.shared_out != nullptr) {
                const uint32_t ss[4] = { sh[c].x, sh[c].y, sh[c].z, sh[c].w };
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[c][2 * j] += gate * bf16_bits_to_f32(ss[j] & 0xffffu);
                    acc[c][2 * j + 1] += gate * bf16_bits_to_f32(ss[j] >> 16);
                }
            }
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 r2 = __floats2bfloat162_rn(acc[c][2 * j], acc[c][2 * j + 1]);
                o[j] = *reinterpret_cast<const uint32_t*>(&r2);
            }
            out[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// dst_j[r * bytes_j ...] = peer block r, segment j: every rank copies the token blocks of all
// ranks (its own included) out of the ranks' symmetric buffers with plain 16-byte peer loads.
// Grid: (chunks, ranks, segments).
__global__ void __launch_bounds__(256) ep_pull_tokens_kernel(EpPullTokensParams p)
{
    const uint32_t r = blockIdx.y, seg = blockIdx.z;
    const uint64_t vecs = p.seg_bytes[seg] / 16;
    const uint4* src = reinterpret_cast<const uint4*>(p.peer[r] + p.seg_offset[seg]);
    uint4* dst = reinterpret_cast<uint4*>(p.dst[seg] + static_cast<uint64_t>(r) * p.seg_bytes[seg]);
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i0 = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < vecs; i0 += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (i0 + q * stride < vecs)
                v[q] = src[i0 + q * stride];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (i0 + q * stride < vecs)
                dst[i0 + q * stride] = v[q];
    }
}

} // namespace

cudaError_t launch_ep_pull_combine(const EpPullParams& params, cudaStream_t stream)
{
    if (params.num_tokens == 0)
        return cudaSuccess;
    EpPullParams p = params;
    static const uint32_t dbg = [] {
        const char* v = std::getenv("QS3_EP_FINISH_DBG");
        return v != nullptr ? static_cast<uint32_t>(std::atoi(v)) : 0u;
    }();
    p.dbg = dbg;
    ep_pull_combine_kernel<<<(p.num_tokens + kEpTokensPerBlock - 1) / kEpTokensPerBlock, 64 * kEpTokensPerBlock, 0,
                             stream>>>(p);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_ep_pull_tokens(const EpPullTokensParams& p, cudaStream_t stream)
{
    if (p.num_ranks == 0 || p.num_segments == 0)
        return cudaSuccess;
    uint64_t largest = 0;
    for (uint32_t j = 0; j < p.num_segments; ++j)
        largest = std::max<uint64_t>(largest, p.seg_bytes[j]);
    const uint32_t chunks = static_cast<uint32_t>(std::min<uint64_t>(2 * 148, std::max<uint64_t>(1, largest / 16 / 1024)));
    ep_pull_tokens_kernel<<<dim3(chunks, p.num_ranks, p.num_segments), 256, 0, stream>>>(p);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_ep_route_targets(const int32_t* ids, const int32_t* map, uint32_t map_len, int32_t* out,
                                    uint32_t* mask, uint32_t tokens, uint32_t top_k, uint32_t per_rank,
                                    uint32_t ranks, cudaStream_t stream)
{
    if (tokens == 0 || (map == nullptr && mask == nullptr))
        return cudaSuccess;
    ep_route_targets_kernel<<<(tokens + 255) / 256, 256, 0, stream>>>(ids, map, map_len, out, mask, tokens, top_k,
                                                                      per_rank, ranks);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_ep_pull_routed(const EpPullRoutedParams& p, cudaStream_t stream)
{
    if (p.num_ranks == 0 || p.num_tokens == 0)
        return cudaSuccess;
    const uint32_t groups = (p.num_tokens + 7) / 8 * p.num_ranks;
    ep_pull_routed_kernel<<<(groups + 7) / 8, 256, 0, stream>>>(p);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_ep_rank_routes(int32_t* rows, float* weights, uint32_t tokens, uint32_t ranks,
                                  cudaStream_t stream)
{
    const uint32_t total = tokens * ranks;
    ep_rank_routes_kernel<<<(total + 255) / 256, 256, 0, stream>>>(rows, weights, tokens, ranks);
    note_launch();
    return cudaGetLastError();
}

size_t route_tables_carve(char* base, uint32_t routes, uint32_t experts, RouteTables* out, uint32_t tile_rows)
{
    RouteTables rt {};
    size_t off = 0;
    const uint64_t seg = routes < experts ? routes : experts; // experts that can hold a row
    const uint64_t max_pad_rows = align_up(routes, tile_rows) + seg * tile_rows;
    rt.tile_rows = tile_rows;
    rt.max_pad_rows = static_cast<uint32_t>(max_pad_rows);
    rt.max_tiles = static_cast<uint32_t>(max_pad_rows / tile_rows);
    rt.route_blocks = (routes + kSortChunk - 1) / kSortChunk;
    rt.counts = carve<int32_t>(base, off, experts);
    rt.indptr = carve<int32_t>(base, off, experts + 1);
    rt.pad_indptr = carve<int32_t>(base, off, experts + 1);
    rt.route_rows = carve<int32_t>(base, off, routes);
    rt.route_prows = carve<int32_t>(base, off, routes);
    rt.row_tokens = carve<int32_t>(base, off, routes);
    rt.row_scales = carve<float>(base, off, routes);
    rt.tile_expert = carve<int32_t>(base, off, rt.max_tiles);
    rt.tile_row0 = carve<int32_t>(base, off, rt.max_tiles);
    rt.tile_nrows = carve<int32_t>(base, off, rt.max_tiles);
    rt.total_tiles = carve<int32_t>(base, off, 1);
    if (tile_rows == static_cast<uint32_t>(kTileM)) {
        rt.pair_expert = carve<int32_t>(base, off, rt.max_tiles);
        rt.pair_row0 = carve<int32_t>(base, off, rt.max_tiles);
        rt.pair_nrows = carve<int32_t>(base, off, rt.max_tiles);
        rt.pair_counts = carve<int32_t>(base, off, 2);
    }
    rt.block_hist = carve<int32_t>(base, off, static_cast<size_t>(rt.route_blocks) * experts);
    if (out != nullptr)
        *out = rt;
    return align_up(off, kWorkspaceAlign);
}

size_t route_tables_bytes(uint32_t routes, uint32_t experts)
{
    return route_tables_carve(nullptr, routes, experts, nullptr);
}

cudaError_t launch_route_sort(const int32_t* topk_ids, const float* topk_weights, uint32_t routes,
                              uint32_t top_k, uint32_t local_offset, uint32_t experts,
                              const RouteTables& rt, cudaStream_t stream)
{
    const size_t smem = static_cast<size_t>(kSortWarps) * experts * sizeof(uint16_t);
    if (smem > 200 * 1024)
        return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(route_hist_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
        if (err == cudaSuccess)
            err = cudaFuncSetAttribute(route_place_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
        if (err != cudaSuccess)
            return err;
    }
    if (rt.route_blocks <= kSmallSortChunks && rt.route_blocks * smem <= 96 * 1024) {
        const size_t small_smem = rt.route_blocks * smem;
        if (small_smem > 48 * 1024) {
            cudaError_t aerr = cudaFuncSetAttribute(route_sort_small_kernel,
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    static_cast<int>(96 * 1024));
            if (aerr != cudaSuccess)
                return aerr;
        }
        route_sort_small_kernel<<<1, kSortWarps * 32, small_smem, stream>>>(topk_ids, topk_weights, routes, top_k,
                                                                           local_offset, experts, rt);
        note_launch();
        return cudaGetLastError();
    }
    route_hist_kernel<<<rt.route_blocks, kSortWarps * 32, smem, stream>>>(
        topk_ids, routes, local_offset, experts, rt.block_hist);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
        return err;
    route_scan_kernel<<<1, 1024, 0, stream>>>(rt.block_hist, rt.route_blocks, experts, rt);
    err = cudaGetLastError();
    if (err != cudaSuccess)
        return err;
    route_place_kernel<<<rt.route_blocks, kSortWarps * 32, smem, stream>>>(
        topk_ids, topk_weights, routes, top_k, local_offset, experts, rt);
    note_launch(3);
    return cudaGetLastError();
}

cudaError_t launch_gather_rows(const void* src, uint32_t row_bytes, const int32_t* route_prows, uint32_t routes,
                               uint32_t top_k, void* dst, cudaStream_t stream)
{
    if (row_bytes % 4 != 0)
        return cudaErrorInvalidValue;
    const bool vec16 = row_bytes % 16 == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    if (vec16)
        gather_bf16_kernel<<<(routes + 7) / 8, 256, 0, stream>>>(static_cast<const uint4*>(src), route_prows, routes,
                                                                top_k, row_bytes / 16, static_cast<uint4*>(dst));
    else
        gather_words_kernel<<<(routes + 7) / 8, 256, 0, stream>>>(static_cast<const uint32_t*>(src), route_prows,
                                                                 routes, top_k, row_bytes / 4,
                                                                 static_cast<uint32_t*>(dst));
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_gather_bf16(const __nv_bfloat16* hidden, const int32_t* route_prows,
                               uint32_t routes, uint32_t top_k, uint32_t hidden_size,
                               __nv_bfloat16* expanded, cudaStream_t stream)
{
    gather_bf16_kernel<<<(routes + 7) / 8, 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(hidden), route_prows, routes, top_k, hidden_size / 8,
        reinterpret_cast<uint4*>(expanded));
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_combine(const CombineParams& p, cudaStream_t stream)
{
    if (p.num_tokens == 0)
        return cudaSuccess;
    const uint32_t blocks = (p.num_tokens + kCombineTokens - 1) / kCombineTokens;
    if (p.residual != nullptr) {
        if (p.hidden_size > 4 * kCombineGroup * 8 || p.skip_empty)
            return cudaErrorNotSupported;
        combine_norm_kernel<<<blocks, kCombineTokens * kCombineGroup, 0, stream>>>(p);
    } else {
        combine_kernel<<<blocks, kCombineTokens * kCombineGroup, 0, stream>>>(p);
    }
    note_launch();
    return cudaGetLastError();
}

} // namespace qs3

// ---- route sort without any allocation ------------------------------------------------
//
// qs3_moe_route_sort_static runs the same three counting-sort kernels as the MoE
// execute calls, but takes its scratch (block histograms, padded segment starts, tile
// table) from the fixed array below instead of a caller workspace. It is meant for
// callers that cannot obtain device memory at the point where they need the routing
// tables: a serving process that handed its whole HBM budget to weight and cache pools
// at start-up and forbids later cudaMalloc, or code inside a latency-critical or
// stream-ordered section where cudaMalloc's implicit device-wide synchronisation is
// not acceptable. The price is a hard size limit and a buffer that every device
// loading this library keeps until the process exits.
namespace {

constexpr size_t kStaticScratchBytes = QS3_ROUTE_SORT_STATIC_SCRATCH_BYTES;

// Device-resident scratch. In HOST code this name is only a handle for the runtime's
// symbol table, not a device address: kernels must be given the pointer that
// cudaGetSymbolAddress returns (looked up once per device below).
static __device__ __align__(256) unsigned char g_route_sort_scratch[kStaticScratchBytes];

// Per-device address of g_route_sort_scratch, resolved with that device current.
cudaError_t static_scratch_base(unsigned char** out)
{
    static std::mutex mu;
    static unsigned char* base[64] = {};
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess)
        return err;
    if (dev < 0 || dev >= 64)
        return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (base[dev] == nullptr) {
        unsigned char* ptr = nullptr;
        err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_route_sort_scratch);
        if (err != cudaSuccess)
            return err;
        if (ptr == nullptr)
            return cudaErrorInvalidSymbol;
        base[dev] = ptr;
    }
    *out = base[dev];
    return cudaSuccess;
}

template <typename T> T* static_take(unsigned char* base, size_t& offset, size_t count)
{
    offset = qs3::align_up(offset, qs3::kWorkspaceAlign);
    T* p = reinterpret_cast<T*>(base + offset);
    offset += count * sizeof(T);
    return p;
}

bool bad_out(const qsfi_tensor1& t, qsfi_dtype dtype, uint64_t count)
{
    return t.data == nullptr || t.dtype != dtype || t.stride[0] != 1 || t.shape[0] < 0
        || static_cast<uint64_t>(t.shape[0]) < count || (reinterpret_cast<uintptr_t>(t.data) & 3u) != 0;
}

} // namespace

extern "C" qsfi_status qs3_moe_route_sort_static(qsfi_context* ctx, const qs3_route_sort_static_desc* d)
{
    using namespace qs3;
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d == nullptr)
        return set_invalid_arg(ctx, "desc is null");
    if (d->num_tokens == 0 || d->top_k == 0 || d->local_num_experts == 0)
        return set_invalid_arg(ctx, "route sort dimensions must be non-zero");
    const uint64_t routes64 = static_cast<uint64_t>(d->num_tokens) * d->top_k;
    if (routes64 > QS3_ROUTE_SORT_STATIC_MAX_ROUTES || d->local_num_experts > QS3_ROUTE_SORT_STATIC_MAX_EXPERTS)
        return set_unsupported(
            ctx,
            "qs3_moe_route_sort_static handles at most %u routes and %u local experts (got %llu and %u); "
            "use an execute call with a caller workspace for larger problems",
            QS3_ROUTE_SORT_STATIC_MAX_ROUTES, QS3_ROUTE_SORT_STATIC_MAX_EXPERTS,
            static_cast<unsigned long long>(routes64), d->local_num_experts);
    const uint32_t routes = static_cast<uint32_t>(routes64);
    const uint32_t experts = d->local_num_experts;
    if (d->topk_ids.data == nullptr || d->topk_ids.dtype != QSFI_DTYPE_I32 || !contiguous2(d->topk_ids)
        || d->topk_ids.shape[0] != d->num_tokens || d->topk_ids.shape[1] != d->top_k)
        return set_invalid_arg(ctx, "topk_ids must be a contiguous i32 [num_tokens, top_k] tensor");
    if (d->topk_weights.data == nullptr || d->topk_weights.dtype != QSFI_DTYPE_F32
        || !contiguous2(d->topk_weights) || d->topk_weights.shape[0] != d->num_tokens
        || d->topk_weights.shape[1] != d->top_k)
        return set_invalid_arg(ctx, "topk_weights must be a contiguous f32 [num_tokens, top_k] tensor");
    if (bad_out(d->counts, QSFI_DTYPE_I32, experts) || bad_out(d->indptr, QSFI_DTYPE_I32, experts + 1ull)
        || bad_out(d->route_rows, QSFI_DTYPE_I32, routes) || bad_out(d->row_tokens, QSFI_DTYPE_I32, routes)
        || bad_out(d->row_scales, QSFI_DTYPE_F32, routes))
        return set_invalid_arg(ctx, "route sort outputs must be contiguous i32/f32 vectors of the documented length");

    unsigned char* base = nullptr;
    cudaError_t err = static_scratch_base(&base);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "cudaGetSymbolAddress(route sort scratch)");

    // caller-owned outputs + scratch-owned internals; every scratch word that a kernel
    // reads is written earlier in the same call, so nothing needs clearing between calls
    RouteTables rt {};
    size_t off = 0;
    const uint64_t seg = routes < experts ? routes : experts;
    rt.tile_rows = kTileM;
    rt.max_pad_rows = static_cast<uint32_t>(align_up(routes, kTileM) + seg * kTileM);
    rt.max_tiles = rt.max_pad_rows / kTileM;
    rt.route_blocks = (routes + kSortChunk - 1) / kSortChunk;
    rt.counts = static_cast<int32_t*>(d->counts.data);
    rt.indptr = static_cast<int32_t*>(d->indptr.data);
    rt.route_rows = static_cast<int32_t*>(d->route_rows.data);
    rt.row_tokens = static_cast<int32_t*>(d->row_tokens.data);
    rt.row_scales = static_cast<float*>(d->row_scales.data);
    rt.pad_indptr = static_take<int32_t>(base, off, experts + 1ull);
    rt.route_prows = static_take<int32_t>(base, off, routes);
    rt.tile_expert = static_take<int32_t>(base, off, rt.max_tiles);
    rt.tile_row0 = static_take<int32_t>(base, off, rt.max_tiles);
    rt.tile_nrows = static_take<int32_t>(base, off, rt.max_tiles);
    rt.total_tiles = static_take<int32_t>(base, off, 1);
    rt.block_hist = static_take<int32_t>(base, off, static_cast<size_t>(rt.route_blocks) * experts);
    if (off > kStaticScratchBytes)
        return set_unsupported(ctx, "route sort scratch need of %llu bytes exceeds the static %llu bytes",
                               static_cast<unsigned long long>(off),
                               static_cast<unsigned long long>(kStaticScratchBytes));
    err = launch_route_sort(static_cast<const int32_t*>(d->topk_ids.data),
                            static_cast<const float*>(d->topk_weights.data), routes, d->top_k,
                            d->local_expert_offset, experts, rt, ctx->stream);
    return set_cuda_error(ctx, err, "qs3_moe_route_sort_static");
}
