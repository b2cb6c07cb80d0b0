// NVFP4 quantisers and scale-layout kernels: weight preparation (the layout the
// upstream weight loader never produced, src/weight_loader.rs:33-66), activation
// quantisation fused with the token gather, and linear -> tiled scale re-tiling.
#include "common.cuh"
#include "nvfp4.cuh"

namespace qs3 {

namespace {

__device__ __forceinline__ void load16_bf16(const __nv_bfloat16* src, float* x)
{
    const uint4 a = reinterpret_cast<const uint4*>(src)[0];
    const uint4 b = reinterpret_cast<const uint4*>(src)[1];
    const uint32_t w[8] = { a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w };
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        x[2 * i] = bf16_bits_to_f32(w[i] & 0xffffu);
        x[2 * i + 1] = bf16_bits_to_f32(w[i] >> 16);
    }
}

// amax per expert: non-negative floats order like their bit patterns.
__global__ void expert_amax_kernel(const __nv_bfloat16* __restrict__ w, uint64_t per_expert,
                                   uint32_t* __restrict__ amax_bits)
{
    const uint32_t e = blockIdx.y;
    const __nv_bfloat16* we = w + static_cast<uint64_t>(e) * per_expert;
    float m = 0.0f;
    for (uint64_t i = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < per_expert;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x * 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(we + i);
        const uint32_t ws[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            m = fmaxf(m, fabsf(bf16_bits_to_f32(ws[j] & 0xffffu)));
            m = fmaxf(m, fabsf(bf16_bits_to_f32(ws[j] >> 16)));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0)
        atomicMax(amax_bits + e, __float_as_uint(m));
}

__global__ void finish_global_scale_kernel(uint32_t* amax_bits, uint32_t experts)
{
    const uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= experts)
        return;
    const float amax = __uint_as_float(amax_bits[e]);
    const float g = amax > 0.0f ? __fdiv_rn(amax, 6.0f * 448.0f) : 1.0f;
    amax_bits[e] = __float_as_uint(g);
}

// One thread per 16-element block of one weight row.
__global__ void quantize_weight_kernel(const __nv_bfloat16* __restrict__ w, uint32_t rows, uint32_t k,
                                       uint64_t total_blocks, const float* __restrict__ global_scale,
                                       uint8_t* __restrict__ packed, uint8_t* __restrict__ scale_linear,
                                       uint8_t* __restrict__ scale_tiled, uint64_t tiled_bytes, int gated)
{
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_blocks)
        return;
    const uint32_t kb_per_row = k / 16;
    const uint32_t kb = static_cast<uint32_t>(idx % kb_per_row);
    const uint64_t grow = idx / kb_per_row;       // expert * rows + row
    const uint32_t e = static_cast<uint32_t>(grow / rows);
    const uint32_t row = static_cast<uint32_t>(grow % rows);
    float x[16];
    load16_bf16(w + grow * k + static_cast<uint64_t>(kb) * 16, x);
    uint32_t lo, hi;
    const uint8_t code = quantize_block16(x, global_scale[e], &lo, &hi);
    *reinterpret_cast<uint2*>(packed + grow * (k / 2) + static_cast<uint64_t>(kb) * 8) = make_uint2(lo, hi);
    if (scale_linear != nullptr)
        scale_linear[grow * kb_per_row + kb] = code;
    if (scale_tiled != nullptr) {
        const uint64_t tr = gated ? gated_tiled_row(row, rows / 2) : row;
        scale_tiled[static_cast<uint64_t>(e) * tiled_bytes + tiled_scale_offset(tr, kb, k / 64)] = code;
    }
}

// Activation rows to the declared (linear) layout; one thread per block.
__global__ void quantize_act_linear_kernel(const __nv_bfloat16* __restrict__ x, uint32_t k,
                                           uint64_t total_blocks, float g, uint8_t* __restrict__ packed,
                                           uint8_t* __restrict__ scale_linear)
{
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_blocks)
        return;
    float v[16];
    load16_bf16(x + idx * 16, v);
    uint32_t lo, hi;
    const uint8_t code = quantize_block16(v, g, &lo, &hi);
    *reinterpret_cast<uint2*>(packed + idx * 8) = make_uint2(lo, hi);
    scale_linear[idx] = code;
}

// Gather + quantise: one thread per (route, 64-element k group). Reads 128 bytes of
// the token's bf16 row, writes 32 bytes of codes into the padded permuted layout
// and one 32-bit word of four scales into the tiled scale buffer.
__global__ void __launch_bounds__(256)
gather_quantize_kernel(const __nv_bfloat16* __restrict__ hidden, const int32_t* __restrict__ route_prows,
                       uint64_t total, uint32_t top_k, uint32_t hidden_size, float g,
                       uint8_t* __restrict__ packed, uint8_t* __restrict__ scale_tiled)
{
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total)
        return;
    const uint32_t kgroups = hidden_size / 64;
    const uint32_t kg = static_cast<uint32_t>(idx % kgroups);
    const uint32_t route = static_cast<uint32_t>(idx / kgroups);
    // no permutation table: rows stay in token order (dense quantisation)
    const int prow = route_prows != nullptr ? route_prows[route] : static_cast<int>(route);
    if (prow < 0)
        return;
    const __nv_bfloat16* src = hidden + static_cast<uint64_t>(route / top_k) * hidden_size + kg * 64;
    uint32_t words[8];
    uint32_t sf = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        float x[16];
        load16_bf16(src + b * 16, x);
        const uint8_t code = quantize_block16(x, g, &words[2 * b], &words[2 * b + 1]);
        sf |= static_cast<uint32_t>(code) << (8 * b);
    }
    uint4* dst = reinterpret_cast<uint4*>(packed + static_cast<uint64_t>(prow) * (hidden_size / 2) + kg * 32);
    dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
    dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
    *reinterpret_cast<uint32_t*>(scale_tiled + tiled_scale_offset(prow, 4ull * kg, kgroups)) = sf;
}

// Gather of already-quantised rows (declared layout) into the padded permuted
// layout; scales move from linear [T, H/16] to tiled. One thread per (route, k group).
__global__ void __launch_bounds__(256)
gather_packed_kernel(const uint8_t* __restrict__ hidden_packed, const uint8_t* __restrict__ hidden_scale,
                     const int32_t* __restrict__ route_prows, uint64_t total, uint32_t top_k,
                     uint32_t hidden_size, uint8_t* __restrict__ packed, uint8_t* __restrict__ scale_tiled,
                     int src_scale_tiled)
{
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total)
        return;
    const uint32_t kgroups = hidden_size / 64;
    const uint32_t kg = static_cast<uint32_t>(idx % kgroups);
    const uint32_t route = static_cast<uint32_t>(idx / kgroups);
    const int prow = route_prows[route];
    if (prow < 0)
        return;
    const uint64_t token = route / top_k;
    const uint4* src = reinterpret_cast<const uint4*>(hidden_packed + token * (hidden_size / 2) + kg * 32);
    uint4* dst = reinterpret_cast<uint4*>(packed + static_cast<uint64_t>(prow) * (hidden_size / 2) + kg * 32);
    dst[0] = src[0];
    dst[1] = src[1];
    // source scales: row-major [T, H/16], or already tiled by token row
    const uint64_t src_off = src_scale_tiled ? tiled_scale_offset(token, 4ull * kg, kgroups)
                                             : token * (hidden_size / 16) + kg * 4;
    const uint32_t sf = *reinterpret_cast<const uint32_t*>(hidden_scale + src_off);
    *reinterpret_cast<uint32_t*>(scale_tiled + tiled_scale_offset(prow, 4ull * kg, kgroups)) = sf;
}

// The same gather organised by destination tile, for 128-row token tiles: block (k chunk, tile)
// moves the rows of one token tile of one expert for 512 elements of k. The codes of a row chunk are 256 contiguous
// bytes (16 threads x 16 bytes), and a scale tile of the destination (512 bytes: 32 lanes x
// four 32-row groups) is written with one 16-byte store per lane instead of 128 scattered
// 4-byte stores. Rows are found through the
// routing tables: padded row -> dense row -> token.
constexpr uint32_t kGatherChunk = 512; // elements of k per block

__global__ void __launch_bounds__(256)
gather_packed_tiles_kernel(const uint8_t* __restrict__ hidden_packed, const uint8_t* __restrict__ hidden_scale,
                           const RouteTables rt, uint32_t hidden_size, uint8_t* __restrict__ packed,
                           uint8_t* __restrict__ scale_tiled, int src_scale_tiled)
{
    const uint32_t tile = blockIdx.y;
    if (static_cast<int>(tile) >= *rt.total_tiles)
        return;
    const int expert = rt.tile_expert[tile];
    const uint32_t row0 = static_cast<uint32_t>(rt.tile_row0[tile]);
    const uint32_t nrows = static_cast<uint32_t>(rt.tile_nrows[tile]);
    // dense (unpadded) row of the tile's first row: same offset inside the expert's segment
    const uint32_t dense0 = static_cast<uint32_t>(rt.indptr[expert])
        + (row0 - static_cast<uint32_t>(rt.pad_indptr[expert]));
    const uint32_t kgroups = hidden_size / 64;
    const uint32_t row_bytes = hidden_size / 2;
    const uint32_t chunk_bytes = kGatherChunk / 2;
    const uint32_t c0 = blockIdx.x * chunk_bytes;

    // codes: 16 threads per row, 16 rows per pass
    const uint32_t sub = threadIdx.x & 15;
    if (c0 + sub * 16 < row_bytes) {
        for (uint32_t j = threadIdx.x >> 4; j < nrows; j += 16) {
            const uint64_t token = static_cast<uint64_t>(rt.row_tokens[dense0 + j]);
            const uint4 v = *reinterpret_cast<const uint4*>(hidden_packed + token * row_bytes + c0 + sub * 16);
            *reinterpret_cast<uint4*>(packed + static_cast<uint64_t>(row0 + j) * row_bytes + c0 + sub * 16) = v;
        }
    }
    // scales: this block's k groups
    const uint32_t kg0 = blockIdx.x * (kGatherChunk / 64);
    const auto src_word = [&](uint32_t j, uint32_t kg) -> uint32_t {
        if (j >= nrows)
            return 0u;
        const uint64_t token = static_cast<uint64_t>(rt.row_tokens[dense0 + j]);
        const uint64_t off = src_scale_tiled ? tiled_scale_offset(token, 4ull * kg, kgroups)
                                             : token * (hidden_size / 16) + kg * 4;
        return *reinterpret_cast<const uint32_t*>(hidden_scale + off);
    };
    // thread = (k group, lane of the scale tile): the words of rows lane, lane + 32, lane + 64, lane + 96
    const uint32_t kg = kg0 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (kg < kgroups) {
        const uint4 v = make_uint4(src_word(lane, kg), src_word(lane + 32, kg), src_word(lane + 64, kg),
                                   src_word(lane + 96, kg));
        *reinterpret_cast<uint4*>(scale_tiled + (static_cast<uint64_t>(row0 >> 7) * kgroups + kg) * 512 + lane * 16)
            = v;
    }
}

// linear [experts, rows, k/16] -> tiled; one thread per (row, k group).
__global__ void tile_scales_kernel(const uint8_t* __restrict__ linear, uint32_t rows, uint32_t k,
                                   uint64_t total, uint8_t* __restrict__ tiled, uint64_t tiled_bytes,
                                   int gated)
{
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total)
        return;
    const uint32_t kgroups = k / 64;
    const uint32_t kg = static_cast<uint32_t>(idx % kgroups);
    const uint64_t grow = idx / kgroups;
    const uint32_t e = static_cast<uint32_t>(grow / rows);
    const uint32_t row = static_cast<uint32_t>(grow % rows);
    const uint32_t sf = *reinterpret_cast<const uint32_t*>(linear + grow * (k / 16) + kg * 4);
    const uint64_t tr = gated ? gated_tiled_row(row, rows / 2) : row;
    *reinterpret_cast<uint32_t*>(tiled + static_cast<uint64_t>(e) * tiled_bytes
                                 + tiled_scale_offset(tr, 4ull * kg, kgroups))
        = sf;
}

uint32_t blocks_for(uint64_t total, uint32_t threads)
{
    return static_cast<uint32_t>((total + threads - 1) / threads);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

} // namespace

cudaError_t launch_nvfp4_gather_quantize(const __nv_bfloat16* hidden, const int32_t* route_prows,
                                         uint32_t routes, uint32_t top_k, uint32_t hidden_size,
                                         float global_scale, uint8_t* packed, uint8_t* scale_tiled,
                                         cudaStream_t stream)
{
    const uint64_t total = static_cast<uint64_t>(routes) * (hidden_size / 64);
    gather_quantize_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(
        hidden, route_prows, total, top_k, hidden_size, global_scale == 0.0f ? 1.0f : global_scale, packed,
        scale_tiled);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_nvfp4_gather_packed(const uint8_t* hidden_packed, const uint8_t* hidden_scale,
                                       const int32_t* route_prows, uint32_t routes, uint32_t top_k,
                                       uint32_t hidden_size, uint8_t* packed, uint8_t* scale_tiled,
                                       cudaStream_t stream, int src_scale_tiled)
{
    const uint64_t total = static_cast<uint64_t>(routes) * (hidden_size / 64);
    gather_packed_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(
        hidden_packed, hidden_scale, route_prows, total, top_k, hidden_size, packed, scale_tiled,
        src_scale_tiled);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_nvfp4_gather_tiles(const uint8_t* hidden_packed, const uint8_t* hidden_scale, const RouteTables& rt,
                                      uint32_t routes, uint32_t top_k, uint32_t hidden_size, uint8_t* packed,
                                      uint8_t* scale_tiled, cudaStream_t stream, int src_scale_tiled)
{
    if (rt.max_tiles == 0)
        return cudaSuccess;
    // 32-row tiles (decode batches) hold a few rows each: a thread per (route, k group) does better there
    if (rt.tile_rows != 128)
        return launch_nvfp4_gather_packed(hidden_packed, hidden_scale, rt.route_prows, routes, top_k, hidden_size,
                                          packed, scale_tiled, stream, src_scale_tiled);
    const dim3 grid((hidden_size + kGatherChunk - 1) / kGatherChunk, rt.max_tiles, 1);
    gather_packed_tiles_kernel<<<grid, 256, 0, stream>>>(hidden_packed, hidden_scale, rt, hidden_size, packed,
                                                        scale_tiled, src_scale_tiled);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_tile_scales(const uint8_t* linear, uint32_t experts, uint32_t rows, uint32_t k,
                               int gated, uint8_t* tiled, cudaStream_t stream)
{
    const uint64_t total = static_cast<uint64_t>(experts) * rows * (k / 64);
    tile_scales_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(
        linear, rows, k, total, tiled, qs3_nvfp4_tiled_scale_bytes(rows, k), gated);
    note_launch();
    return cudaGetLastError();
}

} // namespace qs3

using namespace qs3;

extern "C" {

qsfi_status qs3_nvfp4_quantize_weight(qsfi_context* ctx, const qs3_nvfp4_quantize_weight_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d == nullptr)
        return set_invalid_arg(ctx, "desc is null");
    if (d->weight.data == nullptr || d->weight.dtype != QSFI_DTYPE_BF16 || !contiguous3(d->weight))
        return set_invalid_arg(ctx, "weight must be a contiguous bf16 [experts, rows, k] tensor");
    const int64_t experts = d->weight.shape[0], rows = d->weight.shape[1], k = d->weight.shape[2];
    if (experts <= 0 || rows <= 0 || k <= 0 || k % 64 != 0)
        return set_invalid_arg(ctx, "NVFP4 weight quantisation requires k divisible by 64");
    if (d->gated_rows != 0 && rows % 128 != 0)
        return set_invalid_arg(ctx, "gated NVFP4 weights require 2*intermediate divisible by 128");
    if (d->packed.data == nullptr || d->packed.dtype != QSFI_DTYPE_U8 || !contiguous3(d->packed)
        || d->packed.shape[0] != experts || d->packed.shape[1] != rows || d->packed.shape[2] != k / 2)
        return set_invalid_arg(ctx, "packed must be a contiguous u8 [experts, rows, k/2] tensor");
    if (d->global_scale.data == nullptr || d->global_scale.dtype != QSFI_DTYPE_F32
        || d->global_scale.shape[0] != experts || !contiguous1(d->global_scale))
        return set_invalid_arg(ctx, "global_scale must be a contiguous f32 [experts] tensor");
    if (d->scale_linear.data != nullptr
        && (d->scale_linear.dtype != QSFI_DTYPE_FP8_E4M3 || !contiguous3(d->scale_linear)
            || d->scale_linear.shape[0] != experts || d->scale_linear.shape[1] != rows
            || d->scale_linear.shape[2] != k / 16))
        return set_invalid_arg(ctx, "scale_linear must be a contiguous e4m3 [experts, rows, k/16] tensor");
    const uint64_t tiled_bytes = qs3_nvfp4_tiled_scale_bytes(rows, k);
    if (d->scale_tiled.data != nullptr
        && (d->scale_tiled.dtype != QSFI_DTYPE_U8 || !contiguous1(d->scale_tiled)
            || static_cast<uint64_t>(d->scale_tiled.shape[0]) < tiled_bytes * experts))
        return set_invalid_arg(ctx, "scale_tiled is too small");
    if (!aligned16(d->weight.data) || !aligned16(d->packed.data)
        || (d->scale_tiled.data != nullptr && !aligned16(d->scale_tiled.data)))
        return set_invalid_arg(ctx, "NVFP4 quantisation buffers must be 16-byte aligned");

    cudaStream_t st = ctx->stream;
    uint32_t* g = static_cast<uint32_t*>(d->global_scale.data);
    cudaError_t err = cudaMemsetAsync(g, 0, sizeof(uint32_t) * experts, st);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "cudaMemsetAsync global_scale");
    const uint64_t per_expert = static_cast<uint64_t>(rows) * k;
    dim3 grid(static_cast<uint32_t>(std::min<uint64_t>((per_expert / 8 + 255) / 256, 1024)),
              static_cast<uint32_t>(experts));
    expert_amax_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(d->weight.data),
                                              per_expert, g);
    finish_global_scale_kernel<<<blocks_for(experts, 256), 256, 0, st>>>(g, static_cast<uint32_t>(experts));
    if (d->scale_tiled.data != nullptr && rows % 128 != 0) {
        // rows of the last 128-row block that do not exist keep scale 0
        err = cudaMemsetAsync(d->scale_tiled.data, 0, tiled_bytes * experts, st);
        if (err != cudaSuccess)
            return set_cuda_error(ctx, err, "cudaMemsetAsync scale_tiled");
    }
    const uint64_t total = static_cast<uint64_t>(experts) * rows * (k / 16);
    quantize_weight_kernel<<<blocks_for(total, 256), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(d->weight.data), static_cast<uint32_t>(rows),
        static_cast<uint32_t>(k), total, static_cast<const float*>(d->global_scale.data),
        static_cast<uint8_t*>(d->packed.data), static_cast<uint8_t*>(d->scale_linear.data),
        static_cast<uint8_t*>(d->scale_tiled.data), tiled_bytes, d->gated_rows != 0);
    note_launch(3);
    return set_cuda_error(ctx, cudaGetLastError(), "qs3_nvfp4_quantize_weight");
}

qsfi_status qs3_nvfp4_quantize_act(qsfi_context* ctx, const qs3_nvfp4_quantize_act_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d == nullptr)
        return set_invalid_arg(ctx, "desc is null");
    if (d->x.data == nullptr || d->x.dtype != QSFI_DTYPE_BF16 || !contiguous2(d->x)
        || d->x.shape[0] != d->rows || d->x.shape[1] <= 0 || d->x.shape[1] % 16 != 0)
        return set_invalid_arg(ctx, "x must be a contiguous bf16 [rows, k] tensor with k divisible by 16");
    const int64_t k = d->x.shape[1];
    if (d->packed.data == nullptr || d->packed.dtype != QSFI_DTYPE_U8 || !contiguous2(d->packed)
        || d->packed.shape[0] != d->rows || d->packed.shape[1] != k / 2)
        return set_invalid_arg(ctx, "packed must be a contiguous u8 [rows, k/2] tensor");
    if (d->scale_linear.data == nullptr || d->scale_linear.dtype != QSFI_DTYPE_FP8_E4M3
        || !contiguous2(d->scale_linear) || d->scale_linear.shape[0] != d->rows
        || d->scale_linear.shape[1] != k / 16)
        return set_invalid_arg(ctx, "scale_linear must be a contiguous e4m3 [rows, k/16] tensor");
    if (!aligned16(d->x.data) || !aligned16(d->packed.data))
        return set_invalid_arg(ctx, "NVFP4 quantisation buffers must be 16-byte aligned");
    const uint64_t total = static_cast<uint64_t>(d->rows) * (k / 16);
    quantize_act_linear_kernel<<<blocks_for(total, 256), 256, 0, ctx->stream>>>(
        static_cast<const __nv_bfloat16*>(d->x.data), static_cast<uint32_t>(k), total,
        d->global_scale == 0.0f ? 1.0f : d->global_scale, static_cast<uint8_t*>(d->packed.data),
        static_cast<uint8_t*>(d->scale_linear.data));
    note_launch();
    return set_cuda_error(ctx, cudaGetLastError(), "qs3_nvfp4_quantize_act");
}

qsfi_status qs3_nvfp4_tile_scales(qsfi_context* ctx, const qs3_nvfp4_tile_scales_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d == nullptr)
        return set_invalid_arg(ctx, "desc is null");
    if (d->scale_linear.data == nullptr || d->scale_linear.dtype != QSFI_DTYPE_FP8_E4M3
        || !contiguous3(d->scale_linear) || d->scale_linear.shape[2] <= 0
        || d->scale_linear.shape[2] % 4 != 0)
        return set_invalid_arg(ctx, "scale_linear must be a contiguous e4m3 [experts, rows, k/16] tensor with k divisible by 64");
    const int64_t experts = d->scale_linear.shape[0], rows = d->scale_linear.shape[1];
    const int64_t k = d->scale_linear.shape[2] * 16;
    if (d->gated_rows != 0 && rows % 128 != 0)
        return set_invalid_arg(ctx, "gated NVFP4 weights require 2*intermediate divisible by 128");
    const uint64_t tiled_bytes = qs3_nvfp4_tiled_scale_bytes(rows, k);
    if (d->scale_tiled.data == nullptr || d->scale_tiled.dtype != QSFI_DTYPE_U8
        || static_cast<uint64_t>(d->scale_tiled.shape[0]) < tiled_bytes * experts)
        return set_invalid_arg(ctx, "scale_tiled is too small");
    if ((reinterpret_cast<uintptr_t>(d->scale_linear.data) & 3u) != 0 || !aligned16(d->scale_tiled.data))
        return set_invalid_arg(ctx, "scale buffers are misaligned");
    if (rows % 128 != 0) {
        cudaError_t err = cudaMemsetAsync(d->scale_tiled.data, 0, tiled_bytes * experts, ctx->stream);
        if (err != cudaSuccess)
            return set_cuda_error(ctx, err, "cudaMemsetAsync scale_tiled");
    }
    cudaError_t err = launch_tile_scales(static_cast<const uint8_t*>(d->scale_linear.data),
                                         static_cast<uint32_t>(experts), static_cast<uint32_t>(rows),
                                         static_cast<uint32_t>(k), d->gated_rows != 0,
                                         static_cast<uint8_t*>(d->scale_tiled.data), ctx->stream);
    return set_cuda_error(ctx, err, "qs3_nvfp4_tile_scales");
}

} // extern "C"
