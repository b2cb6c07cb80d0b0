// NVFP4 grouped GEMMs for decode-sized batches, where an expert gets a handful of rows.
//
// The prefill kernel (gemm.cu) makes the expert's token rows the M = 128 side of the MMA:
// with three rows per expert 97 % of every instruction multiplies padding, and the tensor
// pipe, not the weight stream, bounds the layer. Here the operands are swapped, as in the FP8
// decode kernel: the 128 WEIGHT rows of a feature block are M, the expert's token tile of 32
// padded rows is N, so one instruction is a quarter of the work and the kernel runs at the
// speed the weights arrive from HBM.
//
//   grid   (feature splits, token tiles); one CTA = one 32-row token tile of one expert and a
//          range of 128-row feature blocks of that expert's weight
//   smem   token panel (all of k: k/256 tiles of 32 x 128 B) resident, its scale tiles (later the
//          gate / up exchange buffer);
//          weight ring: stages x (128 x 128 B codes + 4 scale tiles)
//   TMEM   2 accumulators of 32 columns (lane = feature, column = token) | 2 x 16 columns of
//          weight scales (alternating per k block) | token scales of all of k
//   warps  0-3 epilogue, 4 producer (TMA), 5 MMA issuer
//
// Scale tiles are the library's tiled layout (include/qs3_moe.h): 512 bytes per (128-row
// block, 64-element k group), byte = (row % 32) * 16 + (row / 32 % 4) * 4 + k / 16 % 4, which
// tcgen05.cp.32x128b.warpx4 turns into four TMEM columns, one per group of 32 rows. A token
// tile of 32 rows is one such group. Its scale words are picked out of the tiles in global
// memory by the epilogue warps (idle until the first accumulator is ready) and laid down in
// shared memory as tiles whose group 0 is this token tile, so that the MMA reads them from the
// first column of a 4-column aligned tensor-memory address like any other scale operand.
#include "common.cuh"
#include "nvfp4.cuh"
#include "tcgen05.cuh"

#include <algorithm>

namespace qs3 {
namespace {

using namespace tc;

constexpr int kSwThreads = 192;
constexpr uint32_t kSwTokens = 32;                // token rows per tile = MMA N
constexpr uint32_t kSwPanelTile = kSwTokens * 128; // one k block of the token panel
constexpr uint32_t kSwStageBytes = kTileBytes + kSfBytes;
constexpr uint32_t kSwMaxStages = 8;
constexpr uint32_t kSwMaxKBlocks = 8;             // k <= 2048
constexpr uint32_t kSwMiscBytes = 1024;
constexpr uint32_t kSwUpBytes = 64 * kSwTokens * 4; // gated: up values handed to the gate warps
constexpr uint32_t kSwTmemCols = 256;             // 64 acc + 32 weight scales + <= 128 token scales

enum : uint32_t {
    ERR_SW_PANEL_WAIT = 0x54000001u,
    ERR_SW_FULL_WAIT = 0x54000002u,
    ERR_SW_EMPTY_WAIT = 0x54000003u,
    ERR_SW_ACC_FULL_WAIT = 0x54000004u,
    ERR_SW_ACC_EMPTY_WAIT = 0x54000005u,
};

struct SwapParams {
    uint32_t n;          // output features per group (gated: intermediate size)
    uint32_t k_blocks;   // k / 256
    uint32_t kgroups;    // k / 64
    uint32_t b_rows;     // weight rows per group (gated: 2 n)
    uint32_t num_fb;     // feature blocks: n / 128 (gated: n / 64)
    uint32_t fb_per_cta;
    uint32_t stages;
    const uint8_t* x_sf; // token scales, tiled by padded row
    const uint8_t* w_sf; // weight scales, tiled per group
    uint64_t w_sf_group_stride;
    const int32_t* tile_expert;
    const int32_t* tile_row0;
    const int32_t* tile_nrows;
    const int32_t* total_tiles;
    void* out;           // gated: e2m1 codes [rows, n / 2]; else bf16 [rows, n]
    uint8_t* out_sf;     // gated: tiled scales of the output rows
    float alpha;
    const float* group_scale;
    const float* group_scale_up;
    float out_global;
    uint32_t* err;
};

template <bool GATED>
__global__ void __launch_bounds__(kSwThreads, 2)
gemm_nvfp4_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                       const SwapParams p)
{
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
    constexpr uint32_t kFeat = GATED ? 64 : 128; // output features per feature block

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* panel = smem;                                   // k_blocks x 4 KB
    uint8_t* panel_sf = panel + p.k_blocks * kSwPanelTile;   // kgroups x 512 B
    uint8_t* ring = panel_sf + max((p.kgroups * 512u + 1023u) & ~1023u, GATED ? kSwUpBytes : 0u);
    uint8_t* misc = ring + p.stages * kSwStageBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);
    uint64_t* empty_bar = full_bar + kSwMaxStages;
    uint64_t* acc_full = empty_bar + kSwMaxStages;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* panel_bar = acc_empty + 2;
    uint64_t* sf_bar = panel_bar + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 256);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    // [token][64 features], gated only; reuses the token scale tiles, which are dead once copied to
    // tensor memory (the first accumulator is complete only after those copies)
    float* s_up = reinterpret_cast<float*>(panel_sf);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4); // one arrival per epilogue warp
        }
        mbar_init(panel_bar, 1);
        mbar_init(sf_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kSwTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_wsf = tmem_base + 64;  // 2 x 16 columns
    const uint32_t tmem_xsf = tmem_base + 96;  // kgroups x 4 columns

    if (warp == 4) {
        // ------------------------------------------------------------ producer --
        if (lane == 0) {
            mbar_expect_tx(panel_bar, p.k_blocks * kSwPanelTile);
            for (uint32_t kb = 0; kb < p.k_blocks; ++kb)
                tma_load_2d(panel + kb * kSwPanelTile, &map_x, panel_bar, static_cast<int>(kb * 128), row0);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t fb = fb0; fb < fb1 && ok; ++fb) {
                const int w_row = expert * static_cast<int>(p.b_rows) + static_cast<int>(fb * kFeat);
                const uint8_t* sf_src = p.w_sf + static_cast<uint64_t>(expert) * p.w_sf_group_stride
                    + (static_cast<uint64_t>(fb) * p.kgroups) * 512;
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait<true>(&empty_bar[s], ph ^ 1, abort_flag, p.err, ERR_SW_EMPTY_WAIT)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sb = ring + s * kSwStageBytes;
                    mbar_expect_tx(&full_bar[s], kSwStageBytes);
                    if (GATED) { // 64 gate rows, then the 64 up rows of the same features
                        tma_load_2d(sb, &map_w, &full_bar[s], static_cast<int>(kb * 128), w_row);
                        tma_load_2d(sb + kTileBytes / 2, &map_w, &full_bar[s], static_cast<int>(kb * 128),
                                    w_row + static_cast<int>(p.n));
                    } else {
                        tma_load_2d(sb, &map_w, &full_bar[s], static_cast<int>(kb * 128), w_row);
                    }
                    bulk_load(sb + kTileBytes, sf_src + static_cast<uint64_t>(kb) * kSfBytes, kSfBytes, &full_bar[s]);
                    if (++s == p.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------- MMA issuer --
        if (lane == 0) {
            // M = 128 weight rows, N = 32 tokens, e2m1 x e2m1 with e4m3 block scales, f32 accumulate
            constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((kSwTokens >> 3) << 17) | ((kBM >> 4) << 24);
            bool ok = mbar_wait<true>(panel_bar, 0, abort_flag, p.err, ERR_SW_PANEL_WAIT)
                && mbar_wait<true>(sf_bar, 0, abort_flag, p.err, ERR_SW_PANEL_WAIT);
            if (ok) {
                tc_fence_after();
                for (uint32_t g = 0; g < p.kgroups; ++g)
                    tc_cp_scales(tmem_xsf + 4 * g, scale_desc(smem_u32(panel_sf) + g * 512));
            }
            uint32_t s = 0, ph = 0, sf_flip = 0, u = 0;
            for (uint32_t fb = fb0; fb < fb1 && ok; ++fb, ++u) {
                const uint32_t buf = u & 1;
                if (!mbar_wait<true>(&acc_empty[buf], ((u >> 1) & 1) ^ 1, abort_flag, p.err, ERR_SW_ACC_EMPTY_WAIT)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d = tmem_base + buf * kSwTokens;
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait<true>(&full_bar[s], ph, abort_flag, p.err, ERR_SW_FULL_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sb = smem_u32(ring + s * kSwStageBytes);
                    const uint32_t wsf = tmem_wsf + 16 * sf_flip;
                    sf_flip ^= 1;
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        tc_cp_scales(wsf + 4 * j, scale_desc(sb + kTileBytes + j * 512));
                    const uint64_t da = operand_desc(sb);
                    const uint64_t db = operand_desc(smem_u32(panel + kb * kSwPanelTile));
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        tc_mma_nvfp4(d, da + 2 * j, db + 2 * j, kIdesc, (kb > 0 || j > 0) ? 1u : 0u, wsf + 4 * j,
                                     tmem_xsf + 16 * kb + 4 * j);
                    tc_commit(&empty_bar[s]);
                    if (++s == p.stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok)
                    tc_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue --
        {
            // token scales of this tile: word (row, k group) of the tiled layout -> group 0 of a
            // tile of the same layout in shared memory
            const uint8_t* src = p.x_sf + (static_cast<uint64_t>(row0 >> 7) * p.kgroups) * 512
                + ((static_cast<uint32_t>(row0) >> 5) & 3u) * 4;
            for (uint32_t i = threadIdx.x; i < p.kgroups * 32; i += 128) {
                const uint32_t kg = i >> 5, r = i & 31;
                const uint32_t word = *reinterpret_cast<const uint32_t*>(src + kg * 512 + r * 16);
                *reinterpret_cast<uint4*>(panel_sf + kg * 512 + r * 16) = make_uint4(word, 0u, 0u, 0u);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // tcgen05.cp reads through the async proxy
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 0)
                mbar_arrive(sf_bar);
        }
        const uint32_t lane_base = (warp * 32) << 16;
        float scale = p.alpha == 0.0f ? 1.0f : p.alpha;
        float scale_up = scale;
        if (p.group_scale != nullptr)
            scale *= p.group_scale[expert];
        scale_up *= p.group_scale_up != nullptr ? p.group_scale_up[expert]
                                                : (p.group_scale != nullptr ? p.group_scale[expert] : 1.0f);
        uint32_t u = 0;
        for (uint32_t fb = fb0; fb < fb1; ++fb, ++u) {
            const uint32_t buf = u & 1;
            bool ready = __all_sync(
                0xffffffffu, mbar_wait(&acc_full[buf], (u >> 1) & 1, abort_flag, p.err, ERR_SW_ACC_FULL_WAIT));
            if constexpr (GATED)
                ready = group_all(1, 128, ready); // the four warps meet at barrier 1 below: stop together
            if (!ready)
                break;
            tc_fence_after();
            uint32_t v[kSwTokens];
            tc_ld16(tmem_base + lane_base + buf * kSwTokens, v);
            tc_ld16(tmem_base + lane_base + buf * kSwTokens + 16, v + 16);
            tc_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&acc_empty[buf]);
            if constexpr (GATED) {
                // lanes 0-63 of the tile are gate features, lanes 64-127 the up values of the same
                // features: warps 2 and 3 hand theirs to warps 0 and 1 through shared memory
                if (warp >= 2) {
#pragma unroll
                    for (uint32_t t = 0; t < kSwTokens; ++t)
                        s_up[t * 64 + (warp - 2) * 32 + lane] = __uint_as_float(v[t]) * scale_up;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp < 2) {
                    const uint32_t f = fb * 64 + warp * 32 + lane; // feature of this lane
                    uint8_t* out = static_cast<uint8_t*>(p.out);
                    const uint32_t out_kgroups = p.n / 64;
#pragma unroll
                    for (uint32_t t = 0; t < kSwTokens; ++t) {
                        if (static_cast<int>(t) < nrows) { // uniform across the warp
                            const float g = __uint_as_float(v[t]) * scale;
                            const float a = __fdividef(g, 1.0f + __expf(-g)) * s_up[t * 64 + warp * 32 + lane];
                            // one scale per 16 features = per half warp (same arithmetic as quantize_block16)
                            float amax = fabsf(a);
#pragma unroll
                            for (int m = 1; m < 16; m <<= 1)
                                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
                            const uint8_t code = f32_to_e4m3_sat(__fdiv_rn(__fdiv_rn(amax, 6.0f), p.out_global));
                            const float sc = __fmul_rn(e4m3_to_f32(code), p.out_global);
                            const float q = __fmul_rn(a, sc > 0.0f ? __fdiv_rn(1.0f, sc) : 0.0f);
                            const float q_next = __shfl_down_sync(0xffffffffu, q, 1);
                            const uint64_t prow = static_cast<uint64_t>(row0) + t;
                            if ((lane & 1) == 0) {
                                uint16_t two; // the code pair in both bytes; the first source is the upper nibble
                                asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n\tmov.b16 %0, {b, b};\n\t}"
                                    : "=h"(two)
                                    : "f"(q), "f"(q_next));
                                out[prow * (p.n / 2) + f / 2] = static_cast<uint8_t>(two & 0xffu);
                            }
                            if ((lane & 15) == 0)
                                p.out_sf[tiled_scale_offset(prow, f / 16, out_kgroups)] = code;
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory"); // s_up is reused by the next block
            } else {
                const uint32_t f = fb * 128 + warp * 32 + lane;
                __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
                for (uint32_t t = 0; t < kSwTokens; ++t)
                    if (static_cast<int>(t) < nrows)
                        out[(static_cast<uint64_t>(row0) + t) * p.n + f] = __float2bfloat16(__uint_as_float(v[t]) * scale);
            }
        }
    }

    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kSwTmemCols)
                     : "memory");
    }
}

template <bool GATED>
cudaError_t launch_swap_instance(const CUtensorMap& mw, const CUtensorMap& mx, const SwapParams& sp, dim3 grid,
                                 size_t smem, cudaStream_t stream)
{
    auto kernel = gemm_nvfp4_swap_kernel<GATED>;
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
    kernel<<<grid, kSwThreads, smem, stream>>>(mw, mx, sp);
    note_launch();
    return cudaGetLastError();
}

} // namespace

uint32_t nvfp4_tile_rows(uint32_t routes, uint32_t experts, uint32_t hidden, uint32_t inter)
{
    const bool fits = hidden % 256 == 0 && inter % 256 == 0 && hidden / 256 <= kSwMaxKBlocks
        && inter / 256 <= kSwMaxKBlocks;
    return fits && routes <= 16u * experts ? kSwTokens : static_cast<uint32_t>(kTileM);
}

cudaError_t launch_nvfp4_swap_gemm(const GemmProblem& g, cudaStream_t stream, const char** why)
{
    const auto fail = [&](const char* msg) {
        if (why != nullptr)
            *why = msg;
        return cudaErrorNotSupported;
    };
    const bool gated = g.gated != 0;
    if (g.tile_expert == nullptr || g.tile_rows != kSwTokens)
        return fail("the decode NVFP4 GEMM takes grouped problems with 32-row token tiles");
    if (g.k % 256 != 0 || g.k / 256 > kSwMaxKBlocks || g.n % 128 != 0 || g.n == 0)
        return fail("the decode NVFP4 GEMM needs k divisible by 256 (<= 2048) and n divisible by 128");
    if (gated ? g.epilogue != EPI_SWIGLU_NVFP4 : g.epilogue != EPI_STORE_BF16)
        return fail("the decode NVFP4 GEMM writes NVFP4 SwiGLU rows (gated) or bf16 rows");
    if (g.beta != 0.0f || g.bias != nullptr)
        return fail("the decode NVFP4 GEMM has no beta / bias epilogue");
    if ((reinterpret_cast<uintptr_t>(g.a) & 15u) != 0 || (reinterpret_cast<uintptr_t>(g.b) & 15u) != 0
        || g.a_pitch_bytes != g.k / 2 || g.b_pitch_bytes != g.k / 2)
        return fail("the decode NVFP4 GEMM operands must be contiguous and 16-byte aligned");
    if (g.max_tiles == 0 || g.max_tiles > 65535)
        return fail("the decode NVFP4 GEMM launch grid is too large");

    SwapParams sp {};
    sp.n = g.n;
    sp.k_blocks = g.k / 256;
    sp.kgroups = g.k / 64;
    sp.b_rows = gated ? 2 * g.n : g.n;
    sp.num_fb = gated ? g.n / 64 : g.n / 128;
    sp.x_sf = g.a_scale_tiled;
    sp.w_sf = g.b_scale_tiled;
    sp.w_sf_group_stride = qs3_nvfp4_tiled_scale_bytes(sp.b_rows, g.k);
    sp.tile_expert = g.tile_expert;
    sp.tile_row0 = g.tile_row0;
    sp.tile_nrows = g.tile_nrows;
    sp.total_tiles = g.total_tiles;
    sp.out = g.out;
    sp.out_sf = g.out_scale_tiled;
    sp.alpha = g.alpha;
    sp.group_scale = g.group_scale;
    sp.group_scale_up = g.group_scale_up;
    sp.out_global = g.out_global_scale == 0.0f ? 1.0f : g.out_global_scale;
    sp.err = device_error_word();

    const size_t fixed = 1024 + static_cast<size_t>(sp.k_blocks) * kSwPanelTile
        + std::max((static_cast<size_t>(sp.kgroups) * 512 + 1023) & ~static_cast<size_t>(1023),
                   static_cast<size_t>(gated ? kSwUpBytes : 0))
        + kSwMiscBytes;
    // two CTAs per SM: one CTA's start-up (token panel, scale tiles) hides behind the other's weight stream
    const size_t budget = 112 * 1024;
    sp.stages = static_cast<uint32_t>(std::min<size_t>(kSwMaxStages, (budget - fixed) / kSwStageBytes));
    const size_t smem = fixed + static_cast<size_t>(sp.stages) * kSwStageBytes;

    // feature splits: about eight CTAs per SM over the launch, so that the tail is short
    const uint32_t tiles = std::max(1u, std::min(g.max_tiles, g.est_tiles != 0 ? g.est_tiles : g.max_tiles));
    const uint32_t want = std::max(1u, (8u * device_sm_count() + tiles - 1) / tiles);
    sp.fb_per_cta = std::max(1u, (sp.num_fb + want - 1) / want);
    const uint32_t splits = (sp.num_fb + sp.fb_per_cta - 1) / sp.fb_per_cta;

    CUtensorMap mw, mx;
    if (!make_operand_map(&mw, true, g.b, g.k / 2, static_cast<uint64_t>(g.groups) * sp.b_rows, g.k / 2,
                          gated ? 64 : 128)
        || !make_operand_map(&mx, true, g.a, g.k / 2, g.a_rows, g.k / 2, kSwTokens)) {
        if (why != nullptr)
            *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    const dim3 grid(splits, g.max_tiles, 1);
    return gated ? launch_swap_instance<true>(mw, mx, sp, grid, smem, stream)
                 : launch_swap_instance<false>(mw, mx, sp, grid, smem, stream);
}

} // namespace qs3
