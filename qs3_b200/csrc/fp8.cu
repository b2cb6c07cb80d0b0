// FP8 block-scaled expert path (e4m3 weights with one f32 scale per 128 x 128 block,
// e4m3 activations with one f32 scale per token per 128 elements): quantisers, the
// grouped GEMM on tcgen05 (kind::f8f6f4) and the MoE entry point built on them.
//
// Upstream has no FP8 MoE surface (only the dtype enum values, qs_tensor.h:20-24); the
// conventions are this library's and are restated by the CPU oracle:
//   scale = max(amax / 448, 1e-30);  code = e4m3_rn_sat(x * (1 / scale))
//
// The GEMM is written for decode-sized batches, where a handful of tokens meet each
// expert and the job is to stream the expert weights from HBM once:
//   * operands are swapped: a 128-feature weight tile is the M operand of the MMA and
//     the expert's token tile (NT = 16 or 32 rows) the N operand, so no tensor-core rows
//     are spent on padding tokens;
//   * the token panel [NT, K] stays resident in shared memory, only weights stream
//     through the TMA ring (one 128 x 128-byte tile per stage);
//   * 128 x 128 block scales are not a tcgen05 block-scale format, so every 128-wide k
//     block is accumulated on its own in tensor memory and promoted into f32 registers
//     as acc += partial * (w_scale[block] * x_scale[token, k block]) by the epilogue
//     warps, which run one accumulator buffer behind the MMA issuer (4 buffers).
#include "tcgen05.cuh"

#include <algorithm>

namespace qs3 {

namespace {

using namespace tc;

// ---- quantisers -------------------------------------------------------------------------

__device__ __forceinline__ float fp8_scale_of(float amax)
{
    return fmaxf(__fdiv_rn(amax, 448.0f), 1.0e-30f);
}

__device__ __forceinline__ uint32_t pack_e4m3x4(const float* f, float inv)
{
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        r |= static_cast<uint32_t>(f32_to_e4m3_sat(__fmul_rn(f[i], inv))) << (8 * i);
    return r;
}

// codes[prow, :] / scales[prow, :] = quantise(x[route / top_k, :]); one warp per (route,
// 128-element group), 4 elements per lane. route_prows == NULL: prow = route.
__global__ void __launch_bounds__(256)
fp8_gather_quantize_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ route_prows,
                           uint32_t routes, uint32_t top_k, uint32_t k, uint8_t* __restrict__ codes,
                           float* __restrict__ scales)
{
    const uint32_t groups = k / 128;
    const uint64_t unit = static_cast<uint64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (unit >= static_cast<uint64_t>(routes) * groups)
        return;
    const uint32_t route = static_cast<uint32_t>(unit / groups), g = static_cast<uint32_t>(unit % groups);
    const int prow = route_prows != nullptr ? route_prows[route] : static_cast<int>(route);
    if (prow < 0)
        return;
    const uint2* src = reinterpret_cast<const uint2*>(x + static_cast<size_t>(route / top_k) * k);
    uint32_t* dst = reinterpret_cast<uint32_t*>(codes + static_cast<size_t>(prow) * k);
    const uint2 v = src[g * 32 + lane];
    const float f[4] = { bf16_bits_to_f32(v.x & 0xffffu), bf16_bits_to_f32(v.x >> 16),
                         bf16_bits_to_f32(v.y & 0xffffu), bf16_bits_to_f32(v.y >> 16) };
    float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = fp8_scale_of(amax);
    dst[g * 32 + lane] = pack_e4m3x4(f, __fdiv_rn(1.0f, s));
    if (lane == 0)
        scales[static_cast<size_t>(prow) * groups + g] = s;
}

// One block per (k block, row block, expert): 128 x 128 weights -> codes + one scale.
__global__ void __launch_bounds__(256)
fp8_quantize_weight_kernel(const __nv_bfloat16* __restrict__ w, uint32_t rows, uint32_t k,
                           uint8_t* __restrict__ codes, float* __restrict__ scales)
{
    __shared__ float s_part[8];
    const uint32_t kb = blockIdx.x, rb = blockIdx.y, e = blockIdx.z;
    const uint32_t r = rb * 128 + threadIdx.x / 2;
    const uint32_t c0 = kb * 128 + (threadIdx.x % 2) * 64;
    const bool live = r < rows;
    const size_t off = (static_cast<size_t>(e) * rows + r) * k + c0;
    uint4 v[8];
    float amax = 0.0f;
    if (live) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = reinterpret_cast<const uint4*>(w + off)[i];
            const uint32_t ws[4] = { v[i].x, v[i].y, v[i].z, v[i].w };
#pragma unroll
            for (int j = 0; j < 4; ++j)
                amax = fmaxf(amax, fmaxf(fabsf(bf16_bits_to_f32(ws[j] & 0xffffu)),
                                         fabsf(bf16_bits_to_f32(ws[j] >> 16))));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0)
        s_part[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        amax = fmaxf(amax, s_part[i]);
    const float s = fp8_scale_of(amax);
    const float inv = __fdiv_rn(1.0f, s);
    if (live) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t o[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 q = v[2 * i + h];
                const float f[8] = { bf16_bits_to_f32(q.x & 0xffffu), bf16_bits_to_f32(q.x >> 16),
                                     bf16_bits_to_f32(q.y & 0xffffu), bf16_bits_to_f32(q.y >> 16),
                                     bf16_bits_to_f32(q.z & 0xffffu), bf16_bits_to_f32(q.z >> 16),
                                     bf16_bits_to_f32(q.w & 0xffffu), bf16_bits_to_f32(q.w >> 16) };
                o[2 * h] = pack_e4m3x4(f, inv);
                o[2 * h + 1] = pack_e4m3x4(f + 4, inv);
            }
            reinterpret_cast<uint4*>(codes + off)[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    if (threadIdx.x == 0)
        scales[(static_cast<size_t>(e) * gridDim.y + rb) * gridDim.x + kb] = s;
}

// ---- grouped GEMM -------------------------------------------------------------------------

constexpr int kF8Threads = 192;   // warps 0-3 epilogue, 4 TMA producer, 5 MMA issuer
constexpr int kF8Bufs = 4;        // accumulator buffers in tensor memory
constexpr int kF8MaxStages = 8;
constexpr int kF8MaxKBlocks = 32; // k <= 4096: one weight-scale register per lane
constexpr uint32_t kF8MiscBytes = 256 /* barriers */ + 16 + 4 * 32 * 4 /* amax */ + kF8MaxKBlocks * 32 * 4;

enum : uint32_t {
    ERR_F8_PANEL_WAIT = 0x54000001u,
    ERR_F8_FULL_WAIT = 0x54000002u,
    ERR_F8_EMPTY_WAIT = 0x54000003u,
    ERR_F8_ACC_FULL_WAIT = 0x54000004u,
    ERR_F8_ACC_EMPTY_WAIT = 0x54000005u,
};

struct Fp8Params {
    uint32_t n;            // output features per group (gated: intermediate size); multiple of 128
    uint32_t k_blocks;     // k / 128
    uint32_t b_rows;       // weight rows per group (gated: 2 n)
    uint32_t num_fb;       // n / 128 feature blocks
    uint32_t fb_per_cta;   // feature blocks one CTA walks
    uint32_t stages;       // ring depth
    const float* x_scale;  // [rows, k_blocks]
    const float* w_scale;  // [groups, w_scale_rows, k_blocks]
    uint32_t w_scale_rows; // ceil(b_rows / 128)
    const int32_t* tile_expert;
    const int32_t* tile_row0;
    const int32_t* tile_nrows;
    const int32_t* total_tiles;
    void* out;             // gated: e4m3 codes [rows, n]; else bf16 [rows, n]
    float* out_scale;      // gated: f32 [rows, n / 128]
    uint32_t* err;
};

// Grid: (feature splits, tiles). One CTA: one token tile of one expert (NT padded rows),
// feature blocks [blockIdx.x * fb_per_cta, ...).
//   TMEM: kF8Bufs buffers of (GATED ? 2 : 1) * NT f32 columns (gate columns, then up columns)
//   smem: token panel k_blocks x (NT x 128 B) | ring stages x 16 KB | barriers, scales
template <int NT, bool GATED>
__global__ void __launch_bounds__(kF8Threads)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                const Fp8Params p)
{
    constexpr uint32_t G = GATED ? 2 : 1;
    constexpr uint32_t kAccCols = G * NT;
    constexpr uint32_t kTmemCols = kF8Bufs * kAccCols < 32 ? 32 : kF8Bufs * kAccCols;
    constexpr uint32_t kPanelTile = NT * 128;
    static_assert(NT == 16 || NT == 32, "token tile of 16 or 32 rows");

    const uint32_t tile = blockIdx.y;
    if (static_cast<int>(tile) >= *p.total_tiles)
        return;
    const uint32_t fb0 = blockIdx.x * p.fb_per_cta;
    const uint32_t fb1 = min(p.num_fb, fb0 + p.fb_per_cta);
    if (fb0 >= fb1)
        return;
    const int expert = p.tile_expert[tile];
    const int row0 = p.tile_row0[tile];
    const int nrows = p.tile_nrows[tile];

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* panel = smem;
    uint8_t* ring = panel + ((p.k_blocks * kPanelTile + 1023u) & ~1023u);
    uint8_t* misc = ring + p.stages * kTileBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);
    uint64_t* empty_bar = full_bar + kF8MaxStages;
    uint64_t* acc_full = empty_bar + kF8MaxStages;
    uint64_t* acc_empty = acc_full + kF8Bufs;
    uint64_t* panel_bar = acc_empty + kF8Bufs;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 256);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* s_amax = reinterpret_cast<float*>(misc + 256 + 16);     // [4][NT]
    float* s_xs = s_amax + 4 * 32;                                  // [k_blocks][NT]

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < kF8Bufs; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4); // one arrival per epilogue warp
        }
        mbar_init(panel_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4) {
        // ------------------------------------------------------------ producer --
        if (lane == 0) {
            mbar_expect_tx(panel_bar, p.k_blocks * kPanelTile);
            for (uint32_t kb = 0; kb < p.k_blocks; ++kb)
                tma_load_2d(panel + kb * kPanelTile, &map_x, panel_bar, static_cast<int>(kb * 128), row0);
            uint32_t w = 0;
            bool ok = true;
            for (uint32_t fb = fb0; fb < fb1 && ok; ++fb) {
                const int w_row = expert * static_cast<int>(p.b_rows) + static_cast<int>(fb * 128);
                for (uint32_t kb = 0; kb < p.k_blocks && ok; ++kb) {
#pragma unroll
                    for (uint32_t g = 0; g < G; ++g, ++w) {
                        const uint32_t s = w % p.stages;
                        const uint32_t ph = (w / p.stages) & 1;
                        if (!mbar_wait<true>(&empty_bar[s], ph ^ 1, abort_flag, p.err, ERR_F8_EMPTY_WAIT)) {
                            ok = false;
                            break;
                        }
                        mbar_expect_tx(&full_bar[s], kTileBytes);
                        tma_load_2d(ring + s * kTileBytes, &map_w, &full_bar[s], static_cast<int>(kb * 128),
                                    w_row + static_cast<int>(g * p.n));
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------- MMA issuer --
        if (lane == 0) {
            // M = 128 weight rows, N = NT tokens, e4m3 x e4m3, f32 accumulate, both K-major
            constexpr uint32_t kIdesc = (1u << 4) | ((static_cast<uint32_t>(NT) >> 3) << 17) | ((kBM >> 4) << 24);
            bool ok = mbar_wait<true>(panel_bar, 0, abort_flag, p.err, ERR_F8_PANEL_WAIT);
            uint32_t w = 0, u = 0;
            for (uint32_t fb = fb0; fb < fb1 && ok; ++fb) {
                for (uint32_t kb = 0; kb < p.k_blocks && ok; ++kb, ++u) {
                    const uint32_t buf = u % kF8Bufs;
                    const uint32_t bph = (u / kF8Bufs) & 1;
                    if (!mbar_wait<true>(&acc_empty[buf], bph ^ 1, abort_flag, p.err, ERR_F8_ACC_EMPTY_WAIT)) {
                        ok = false;
                        break;
                    }
                    const uint64_t db = operand_desc(smem_u32(panel + kb * kPanelTile));
#pragma unroll
                    for (uint32_t g = 0; g < G; ++g, ++w) {
                        const uint32_t s = w % p.stages;
                        const uint32_t ph = (w / p.stages) & 1;
                        if (!mbar_wait<true>(&full_bar[s], ph, abort_flag, p.err, ERR_F8_FULL_WAIT)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint64_t da = operand_desc(smem_u32(ring + s * kTileBytes));
                        const uint32_t d = tmem_base + buf * kAccCols + g * NT;
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j)
                            tc_mma_f8(d, da + 2 * j, db + 2 * j, kIdesc, j > 0 ? 1u : 0u);
                        tc_commit(&empty_bar[s]);
                    }
                    if (ok)
                        tc_commit(&acc_full[buf]);
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue --
        // activation scales of the tile: s_xs[kb][t]
        for (uint32_t i = threadIdx.x; i < p.k_blocks * NT; i += 128) {
            const uint32_t kb = i / NT, t = i % NT;
            s_xs[i] = p.x_scale[static_cast<size_t>(row0 + t) * p.k_blocks + kb];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const uint32_t lane_base = (warp * 32) << 16;
        const uint32_t r = warp * 32 + lane; // feature within the block = TMEM lane
        uint32_t u = 0;
        bool ok = true;
        for (uint32_t fb = fb0; fb < fb1 && ok; ++fb) {
            // block scales of this feature block, one k block per lane
            float wsg = 0.0f, wsu = 0.0f;
            if (lane < p.k_blocks) {
                const float* ws = p.w_scale + static_cast<size_t>(expert) * p.w_scale_rows * p.k_blocks;
                wsg = ws[static_cast<size_t>(fb) * p.k_blocks + lane];
                if (GATED)
                    wsu = ws[static_cast<size_t>(p.n / 128 + fb) * p.k_blocks + lane];
            }
            float acc[G][NT];
#pragma unroll
            for (uint32_t g = 0; g < G; ++g)
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    acc[g][t] = 0.0f;
            for (uint32_t kb = 0; kb < p.k_blocks; ++kb, ++u) {
                const uint32_t buf = u % kF8Bufs;
                const uint32_t bph = (u / kF8Bufs) & 1;
                ok = __all_sync(0xffffffffu,
                                mbar_wait(&acc_full[buf], bph, abort_flag, p.err, ERR_F8_ACC_FULL_WAIT));
                if (!ok)
                    break;
                tc_fence_after();
                uint32_t v[G][NT];
#pragma unroll
                for (uint32_t g = 0; g < G; ++g)
#pragma unroll
                    for (int c = 0; c < NT / 16; ++c)
                        tc_ld16(tmem_base + lane_base + buf * kAccCols + g * NT + c * 16, &v[g][c * 16]);
                tc_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&acc_empty[buf]);
                const float sg = __shfl_sync(0xffffffffu, wsg, kb);
                const float su = GATED ? __shfl_sync(0xffffffffu, wsu, kb) : 0.0f;
                const float* xs = s_xs + kb * NT;
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const float x = xs[t];
                    acc[0][t] = fmaf(__uint_as_float(v[0][t]), sg * x, acc[0][t]);
                    if (GATED)
                        acc[G - 1][t] = fmaf(__uint_as_float(v[G - 1][t]), su * x, acc[G - 1][t]);
                }
            }
            if constexpr (GATED)
                ok = group_all(1, 128, ok); // the four warps meet at barrier 1 below: stop together
            if (!ok)
                break;
            const uint32_t f = fb * 128 + r;
            if constexpr (GATED) {
                // SwiGLU, then quantise the tile's 128 features per token (= one scale group)
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const float gte = acc[0][t];
                    acc[0][t] = __fdividef(gte, 1.0f + __expf(-gte)) * acc[1][t];
                    const uint32_t m = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(acc[0][t])));
                    if (lane == 0)
                        s_amax[warp * NT + t] = __uint_as_float(m);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                uint8_t* out = static_cast<uint8_t*>(p.out);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    if (t < nrows) {
                        const float amax = fmaxf(fmaxf(s_amax[t], s_amax[NT + t]),
                                                 fmaxf(s_amax[2 * NT + t], s_amax[3 * NT + t]));
                        const float s = fp8_scale_of(amax);
                        out[static_cast<size_t>(row0 + t) * p.n + f]
                            = f32_to_e4m3_sat(__fmul_rn(acc[0][t], __fdiv_rn(1.0f, s)));
                        if (r == static_cast<uint32_t>(t))
                            p.out_scale[static_cast<size_t>(row0 + t) * p.num_fb + fb] = s;
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory"); // s_amax is reused by the next block
            } else {
                __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    if (t < nrows)
                        out[static_cast<size_t>(row0 + t) * p.n + f] = __float2bfloat16(acc[0][t]);
            }
        }
    }

    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                     : "memory");
    }
}

template <int NT, bool GATED>
cudaError_t launch_fp8_instance(const CUtensorMap& mw, const CUtensorMap& mx, const Fp8Params& fp, dim3 grid,
                                size_t smem, cudaStream_t stream)
{
    auto kernel = gemm_fp8_kernel<NT, GATED>;
    static size_t configured[64] = {}; // largest size set so far, per instantiation and device
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess)
        return err;
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess)
            return err;
        if (dev >= 0 && dev < 64)
            configured[dev] = smem;
    }
    kernel<<<grid, kF8Threads, smem, stream>>>(mw, mx, fp);
    note_launch();
    return cudaGetLastError();
}

} // namespace

uint32_t fp8_tile_rows(uint32_t routes, uint32_t experts)
{
    return routes <= 16u * experts ? 16u : 32u;
}

cudaError_t launch_fp8_gather_quantize(const __nv_bfloat16* x, const int32_t* route_prows, uint32_t routes,
                                       uint32_t top_k, uint32_t k, uint8_t* codes, float* scales,
                                       cudaStream_t stream)
{
    if (routes == 0)
        return cudaSuccess;
    const uint64_t units = static_cast<uint64_t>(routes) * (k / 128);
    fp8_gather_quantize_kernel<<<static_cast<uint32_t>((units + 7) / 8), 256, 0, stream>>>(
        x, route_prows, routes, top_k, k, codes, scales);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_fp8_quantize_weight(const __nv_bfloat16* w, uint32_t experts, uint32_t rows, uint32_t k,
                                       uint8_t* codes, float* scales, cudaStream_t stream)
{
    const dim3 grid(k / 128, (rows + 127) / 128, experts);
    fp8_quantize_weight_kernel<<<grid, 256, 0, stream>>>(w, rows, k, codes, scales);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_fp8_gemm(const Fp8Gemm& g, cudaStream_t stream, const char** why)
{
    const auto fail = [&](const char* msg) {
        if (why != nullptr)
            *why = msg;
        return cudaErrorNotSupported;
    };
    if (g.n % 128 != 0 || g.k % 128 != 0 || g.n == 0 || g.k == 0)
        return fail("FP8 GEMM needs n and k divisible by 128");
    if (g.k / 128 > kF8MaxKBlocks)
        return fail("FP8 GEMM supports k <= 4096");
    if (g.tile_rows != 16 && g.tile_rows != 32)
        return fail("FP8 GEMM token tiles are 16 or 32 rows");
    if ((reinterpret_cast<uintptr_t>(g.x) & 15u) != 0 || (reinterpret_cast<uintptr_t>(g.w) & 15u) != 0)
        return fail("FP8 GEMM operands must be 16-byte aligned");
    Fp8Params fp {};
    fp.n = g.n;
    fp.k_blocks = g.k / 128;
    fp.b_rows = g.gated ? 2 * g.n : g.n;
    fp.num_fb = g.n / 128;
    fp.x_scale = g.x_scale;
    fp.w_scale = g.w_scale;
    fp.w_scale_rows = (fp.b_rows + 127) / 128;
    fp.tile_expert = g.tile_expert;
    fp.tile_row0 = g.tile_row0;
    fp.tile_nrows = g.tile_nrows;
    fp.total_tiles = g.total_tiles;
    fp.out = g.out;
    fp.out_scale = g.out_scale;
    fp.err = device_error_word();

    const size_t panel = (static_cast<size_t>(fp.k_blocks) * g.tile_rows * 128 + 1023) & ~static_cast<size_t>(1023);
    const bool two_per_sm = panel <= 48 * 1024;
    const size_t budget = two_per_sm ? 110 * 1024 : 220 * 1024;
    const size_t fixed = 1024 + panel + kF8MiscBytes;
    if (budget < fixed + 2 * kTileBytes)
        return fail("FP8 GEMM token panel does not fit in shared memory");
    fp.stages = static_cast<uint32_t>(std::min<size_t>(kF8MaxStages, (budget - fixed) / kTileBytes));
    const size_t smem = fixed + static_cast<size_t>(fp.stages) * kTileBytes;

    // feature splits: enough CTAs to fill the resident slots of the device once
    const uint32_t slots = device_sm_count() * (two_per_sm ? 2u : 1u);
    const uint32_t want = std::max(1u, (slots + g.est_tiles - 1) / std::max(1u, g.est_tiles));
    fp.fb_per_cta = std::max(1u, (fp.num_fb + want - 1) / want);
    const uint32_t splits = (fp.num_fb + fp.fb_per_cta - 1) / fp.fb_per_cta;
    if (g.max_tiles == 0 || g.max_tiles > 65535)
        return fail("FP8 GEMM launch grid is too large");

    CUtensorMap mw, mx;
    if (!make_operand_map(&mw, true, g.w, g.k, static_cast<uint64_t>(g.groups) * fp.b_rows, g.k, 128)
        || !make_operand_map(&mx, true, g.x, g.k, g.x_rows, g.k, g.tile_rows)) {
        if (why != nullptr)
            *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    const dim3 grid(splits, g.max_tiles, 1);
    if (g.tile_rows == 16)
        return g.gated ? launch_fp8_instance<16, true>(mw, mx, fp, grid, smem, stream)
                       : launch_fp8_instance<16, false>(mw, mx, fp, grid, smem, stream);
    return g.gated ? launch_fp8_instance<32, true>(mw, mx, fp, grid, smem, stream)
                   : launch_fp8_instance<32, false>(mw, mx, fp, grid, smem, stream);
}

} // namespace qs3
