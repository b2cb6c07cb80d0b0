// Grouped / dense GEMM  D[m, n] = sum_k A[m, k] * B[g][n, k]  on the 5th-generation
// tensor cores (tcgen05), one 128 x 128 output tile per CTA:
//
//   warp 4      TMA producer: A and B tiles (128 rows x 128 bytes, 128-byte swizzle)
//               and, for NVFP4, their scale tiles, into a ring of kStages stages
//   warp 5      allocates tensor memory, issues tcgen05.cp (scales) + tcgen05.mma
//               from one elected lane, frees the ring with tcgen05.commit
//   warps 0-3   epilogue: tcgen05.ld of the f32 accumulator, fused epilogue, stores
//
// A "grouped" problem walks a tile table built by the route sort (one entry per
// 128-row tile of one expert's padded row segment); B is then indexed by the
// tile's expert. "Gated" problems load 64 gate rows and their 64 up rows of B into
// one tile so that the SwiGLU epilogue finds both halves in the same TMEM lane.
// Two CTAs fit on one SM (<= 256 TMEM columns and <= 109 KB shared memory each),
// so one tile's epilogue overlaps the other's main loop.
//
// Every wait is bounded: when a barrier does not flip within ~1 s of SM clocks the
// kernel records a code in the device error word and leaves through the normal
// teardown (tensor memory is freed).
#include "common.cuh"
#include "nvfp4.cuh"

#include <mutex>

namespace qs3 {

namespace {

constexpr int kBM = 128;         // tile rows (tensor-memory lanes)
constexpr int kBN = 128;         // tile columns (accumulator columns)
constexpr int kStages = 3;
constexpr int kTileBytes = 128 * 128; // one operand tile: 128 rows x 128 bytes
constexpr int kSfBytes = 2048;        // scale tile of one stage: 4 k-groups x 512 bytes
constexpr int kThreads = 192;
constexpr uint64_t kWaitCycles = 2000000000ull;

enum : uint32_t {
    ERR_FULL_WAIT = 0x51000001u,
    ERR_EMPTY_WAIT = 0x51000002u,
    ERR_ACC_WAIT = 0x51000003u,
};

struct TcParams {
    uint32_t n;             // output features (gated: gate features)
    uint32_t k_blocks;      // number of 128-byte k blocks
    uint32_t b_rows;        // B rows per group
    uint32_t kgroups;       // k / 64, NVFP4 scale tiling
    const uint8_t* sfa;
    const uint8_t* sfb;
    uint64_t sfb_group_stride;
    const int32_t* tile_expert;
    const int32_t* tile_row0;
    const int32_t* tile_nrows;
    const int32_t* total_tiles;
    uint32_t dense_rows;
    void* out;
    uint64_t out_pitch;     // elements; bytes for packed output
    uint8_t* out_sf;
    uint32_t out_kgroups;   // n / 64 of the quantised output
    float alpha;
    float beta;
    const float* group_scale;
    const float* bias;
    float out_global;
    uint32_t* err;
};

// ---- PTX wrappers -------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}

// Bounded wait; on expiry records `code` and raises the CTA's abort flag.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* err, uint32_t code)
{
    if (mbar_try_wait(bar, parity))
        return true;
    const uint64_t start = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity))
            return true;
        if (*abort_flag != 0)
            return false;
        if (static_cast<uint64_t>(clock64()) - start > kWaitCycles) {
            *abort_flag = 1;
            if (err != nullptr)
                atomicCAS(err, 0u, code);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tc_cp_scales(uint32_t taddr, uint64_t sdesc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void tc_mma_bf16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
                 "l"(a), "l"(b), "r"(idesc), "r"(acc)
                 : "memory");
}

__device__ __forceinline__ void tc_mma_nvfp4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc,
                                             uint32_t sfa, uint32_t sfb)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X"
                 " [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d),
                 "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb)
                 : "memory");
}

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32"
                 " {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                   "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
                   "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand tile stored with the
// 128-byte swizzle: rows are 128 bytes, groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr)
{
    return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(1024 >> 4) << 32)
        | (1ull << 46) | (2ull << 61);
}

// Descriptor of one 512-byte scale tile (32 rows x 16 bytes, no swizzle; groups of
// 8 rows are 128 bytes apart) for tcgen05.cp.32x128b.
__device__ __forceinline__ uint64_t scale_desc(uint32_t smem_addr)
{
    return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(128 >> 4) << 32)
        | (1ull << 46);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b)
{
    const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ float round_bf16(float v)
{
    return __bfloat162float(__float2bfloat16(v));
}

// ---- the kernel ---------------------------------------------------------------------

template <bool NVFP4, bool GATED, int EPI>
__global__ void __launch_bounds__(kThreads)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const TcParams p)
{
    // ---- which tile ----
    const uint32_t tile = blockIdx.y;
    int expert = 0, row0 = 0, nrows = 0;
    if (p.tile_expert != nullptr) {
        if (static_cast<int>(tile) >= *p.total_tiles)
            return;
        expert = p.tile_expert[tile];
        row0 = p.tile_row0[tile];
        nrows = p.tile_nrows[tile];
    } else {
        row0 = static_cast<int>(tile) * kBM;
        nrows = min(kBM, static_cast<int>(p.dense_rows) - row0);
    }
    const uint32_t nt = blockIdx.x;
    constexpr uint32_t kFeat = GATED ? kBN / 2 : kBN; // output features per tile
    const uint32_t n0 = nt * kFeat;

    // ---- shared memory carve-up ----
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr uint32_t kStageBytes = 2 * kTileBytes + (NVFP4 ? 2 * kSfBytes : 0);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* acc_bar = empty_bar + kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    constexpr uint32_t kTmemCols = NVFP4 ? 256 : 128; // accumulator 128 (+ 16 SFA + 16 SFB), power of 2

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_bar, 1);
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
    const uint32_t tmem_sfa = tmem_base + kBN;
    const uint32_t tmem_sfb = tmem_base + kBN + 16;

    if (warp == 4) {
        // ------------------------------------------------------------ producer --
        if (lane == 0) {
            const int b_row = expert * static_cast<int>(p.b_rows) + static_cast<int>(n0);
            const uint8_t* sfa_src = NVFP4
                ? p.sfa + (static_cast<uint64_t>(row0 >> 7) * p.kgroups) * 512
                : nullptr;
            const uint8_t* sfb_src = NVFP4
                ? p.sfb + static_cast<uint64_t>(expert) * p.sfb_group_stride
                    + (static_cast<uint64_t>(nt) * p.kgroups) * 512
                : nullptr;
            for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                const uint32_t s = kb % kStages;
                const uint32_t ph = (kb / kStages) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err, ERR_EMPTY_WAIT))
                    break;
                uint8_t* sa = smem + s * kStageBytes;
                uint8_t* sb = sa + kTileBytes;
                mbar_expect_tx(&full_bar[s], kStageBytes);
                // inner coordinate in elements of the map's type (bf16 elements / bytes)
                const int c0 = static_cast<int>(kb) * (NVFP4 ? 128 : 64);
                tma_load_2d(sa, &map_a, &full_bar[s], c0, row0);
                if (GATED) {
                    tma_load_2d(sb, &map_b, &full_bar[s], c0, b_row);
                    tma_load_2d(sb + kTileBytes / 2, &map_b, &full_bar[s], c0,
                                b_row + static_cast<int>(p.n));
                } else {
                    tma_load_2d(sb, &map_b, &full_bar[s], c0, b_row);
                }
                if (NVFP4) {
                    bulk_load(sb + kTileBytes, sfa_src + static_cast<uint64_t>(kb) * kSfBytes, kSfBytes,
                              &full_bar[s]);
                    bulk_load(sb + kTileBytes + kSfBytes, sfb_src + static_cast<uint64_t>(kb) * kSfBytes,
                              kSfBytes, &full_bar[s]);
                }
            }
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------- MMA issuer --
        if (lane == 0) {
            // instruction descriptor: M = 128, N = 128, both operands K-major
            constexpr uint32_t kIdesc = NVFP4
                ? ((1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24))
                : ((1u << 4) | (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24));
            bool ok = true;
            for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                const uint32_t s = kb % kStages;
                const uint32_t ph = (kb / kStages) & 1;
                if (!mbar_wait(&full_bar[s], ph, abort_flag, p.err, ERR_FULL_WAIT)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * kStageBytes);
                const uint32_t sb = sa + kTileBytes;
                if (NVFP4) {
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        tc_cp_scales(tmem_sfa + 4 * j, scale_desc(sb + kTileBytes + j * 512));
                        tc_cp_scales(tmem_sfb + 4 * j, scale_desc(sb + kTileBytes + kSfBytes + j * 512));
                    }
                }
                const uint64_t da = operand_desc(sa);
                const uint64_t db = operand_desc(sb);
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    // one MMA consumes 32 bytes of K per row: +2 in the 16-byte address field
                    const uint32_t acc = (kb > 0 || j > 0) ? 1u : 0u;
                    if (NVFP4)
                        tc_mma_nvfp4(tmem_base, da + 2 * j, db + 2 * j, kIdesc, acc, tmem_sfa + 4 * j,
                                     tmem_sfb + 4 * j);
                    else
                        tc_mma_bf16(tmem_base, da + 2 * j, db + 2 * j, kIdesc, acc);
                }
                tc_commit(&empty_bar[s]);
            }
            if (ok)
                tc_commit(acc_bar);
        }
    } else {
        // ------------------------------------------------------------ epilogue --
        // warp-uniform: tcgen05.ld below must be executed by whole warps
        const bool ready = __all_sync(0xffffffffu, mbar_wait(acc_bar, 0, abort_flag, p.err, ERR_ACC_WAIT));
        tc_fence_after();
        if (ready) {
            const int r = static_cast<int>(warp * 32 + lane); // tile row = TMEM lane
            const bool row_ok = r < nrows;
            const uint64_t grow = static_cast<uint64_t>(row0) + r;
            const uint32_t lane_base = (warp * 32) << 16;
            float scale = p.alpha == 0.0f ? 1.0f : p.alpha;
            if (p.group_scale != nullptr)
                scale *= p.group_scale[expert];

            if constexpr (!GATED) {
                for (uint32_t c = 0; c < kBN / 16; ++c) {
                    const uint32_t nb = n0 + c * 16;
                    if (nb >= p.n)
                        break;
                    uint32_t v[16];
                    tc_ld16(tmem_base + lane_base + c * 16, v);
                    tc_ld_wait();
                    if (!row_ok)
                        continue;
                    float f[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        f[i] = __uint_as_float(v[i]) * scale;
                    const bool full = nb + 16 <= p.n;
                    if constexpr (EPI == EPI_STORE_F32) {
                        float* o = static_cast<float*>(p.out) + grow * p.out_pitch + nb;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (full || nb + i < p.n) {
                                if (p.beta != 0.0f)
                                    f[i] += p.beta * o[i];
                                if (p.bias != nullptr)
                                    f[i] += p.bias[nb + i];
                            }
                        }
                        if (full && ((reinterpret_cast<uintptr_t>(o) & 15u) == 0)) {
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                reinterpret_cast<float4*>(o)[i]
                                    = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (nb + i < p.n)
                                    o[i] = f[i];
                        }
                    } else {
                        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + grow * p.out_pitch + nb;
                        if (p.beta != 0.0f) {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (full || nb + i < p.n)
                                    f[i] += p.beta * __bfloat162float(o[i]);
                        }
                        if (full && ((reinterpret_cast<uintptr_t>(o) & 15u) == 0)) {
                            uint32_t w[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                w[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
                            reinterpret_cast<uint4*>(o)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            reinterpret_cast<uint4*>(o)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (nb + i < p.n)
                                    o[i] = __float2bfloat16(f[i]);
                        }
                    }
                }
            } else {
                uint32_t sf_word = 0;
                for (uint32_t c = 0; c < kFeat / 16; ++c) {
                    const uint32_t fb = n0 + c * 16; // first gate feature of this chunk
                    if (fb >= p.n)
                        break;
                    uint32_t vg[16], vu[16];
                    tc_ld16(tmem_base + lane_base + c * 16, vg);
                    tc_ld16(tmem_base + lane_base + kFeat + c * 16, vu);
                    tc_ld_wait();
                    if (!row_ok)
                        continue;
                    float act[16];
                    if constexpr (EPI == EPI_SWIGLU_BF16) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            // upstream stores the gate_up product as bf16 before SwiGLU
                            // (qsfi_moe.cu:638-651,445-463)
                            const float g = round_bf16(__uint_as_float(vg[i]) * scale);
                            const float u = round_bf16(__uint_as_float(vu[i]) * scale);
                            act[i] = g * sigmoid_fast(g) * u;
                        }
                        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + grow * p.out_pitch + fb;
                        if (fb + 16 <= p.n && ((reinterpret_cast<uintptr_t>(o) & 15u) == 0)) {
                            uint32_t w[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                w[i] = pack_bf16x2(act[2 * i], act[2 * i + 1]);
                            reinterpret_cast<uint4*>(o)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            reinterpret_cast<uint4*>(o)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (fb + i < p.n)
                                    o[i] = __float2bfloat16(act[i]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float g = __uint_as_float(vg[i]) * scale;
                            const float u = __uint_as_float(vu[i]) * scale;
                            act[i] = g * sigmoid_fast(g) * u;
                        }
                        uint32_t lo, hi;
                        const uint8_t code = quantize_block16(act, p.out_global, &lo, &hi);
                        sf_word |= static_cast<uint32_t>(code) << (8 * c);
                        uint8_t* o = static_cast<uint8_t*>(p.out) + grow * p.out_pitch + fb / 2;
                        *reinterpret_cast<uint2*>(o) = make_uint2(lo, hi);
                    }
                }
                if constexpr (EPI == EPI_SWIGLU_NVFP4) {
                    // the tile's 64 features are exactly one k-group of the next GEMM
                    if (row_ok && n0 < p.n)
                        *reinterpret_cast<uint32_t*>(p.out_sf + tiled_scale_offset(grow, 4ull * nt, p.out_kgroups))
                            = sf_word;
                }
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

// ---- CUDA-core kernel for shapes the tensor-core tiles do not cover ----------------
// (reduction length not a multiple of 8, or operands not 16-byte aligned). One
// thread per output element, f32 accumulation in k order; bf16 operands only.
template <int EPI>
__global__ void gemm_simt_kernel(const __nv_bfloat16* __restrict__ a, uint64_t a_pitch,
                                 const __nv_bfloat16* __restrict__ b, uint64_t b_pitch, TcParams p,
                                 uint32_t k, int gated)
{
    const uint32_t tile = blockIdx.y;
    int expert = 0, row0 = 0, nrows = 0;
    if (p.tile_expert != nullptr) {
        if (static_cast<int>(tile) >= *p.total_tiles)
            return;
        expert = p.tile_expert[tile];
        row0 = p.tile_row0[tile];
        nrows = p.tile_nrows[tile];
    } else {
        row0 = static_cast<int>(tile) * kBM;
        nrows = min(kBM, static_cast<int>(p.dense_rows) - row0);
    }
    float scale = p.alpha == 0.0f ? 1.0f : p.alpha;
    if (p.group_scale != nullptr)
        scale *= p.group_scale[expert];
    const uint32_t cols = blockDim.x; // output features handled per block-row pass
    const uint32_t n = blockIdx.x * cols + threadIdx.x;
    if (n >= p.n)
        return;
    const __nv_bfloat16* bw = b + (static_cast<uint64_t>(expert) * p.b_rows + n) * b_pitch;
    const __nv_bfloat16* bu = bw + static_cast<uint64_t>(p.n) * b_pitch; // up row (gated)
    for (int r = 0; r < nrows; ++r) {
        const uint64_t grow = static_cast<uint64_t>(row0) + r;
        const __nv_bfloat16* ar = a + grow * a_pitch;
        float acc = 0.0f, acc2 = 0.0f;
        for (uint32_t i = 0; i < k; ++i) {
            const float x = __bfloat162float(ar[i]);
            acc += x * __bfloat162float(bw[i]);
            if (gated)
                acc2 += x * __bfloat162float(bu[i]);
        }
        if constexpr (EPI == EPI_SWIGLU_BF16) {
            const float g = round_bf16(acc * scale);
            const float u = round_bf16(acc2 * scale);
            static_cast<__nv_bfloat16*>(p.out)[grow * p.out_pitch + n]
                = __float2bfloat16(g * sigmoid_fast(g) * u);
        } else if constexpr (EPI == EPI_STORE_F32) {
            float* o = static_cast<float*>(p.out) + grow * p.out_pitch + n;
            float v = acc * scale;
            if (p.beta != 0.0f)
                v += p.beta * *o;
            if (p.bias != nullptr)
                v += p.bias[n];
            *o = v;
        } else {
            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + grow * p.out_pitch + n;
            float v = acc * scale;
            if (p.beta != 0.0f)
                v += p.beta * __bfloat162float(*o);
            *o = __float2bfloat16(v);
        }
    }
}

// ---- host side ------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
{
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) == cudaSuccess
            && res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// 2-D map over a row-major [rows, inner] operand; box = 128 bytes x box_rows, 128B swizzle.
bool make_map(CUtensorMap* map, bool bytes_type, const void* base, uint64_t inner_elems, uint64_t rows,
              uint64_t pitch_bytes, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr)
        return false;
    const cuuint64_t dims[2] = { inner_elems, rows };
    const cuuint64_t strides[1] = { pitch_bytes };
    const cuuint32_t box[2] = { bytes_type ? 128u : 64u, box_rows };
    const cuuint32_t estr[2] = { 1, 1 };
    return fn(map, bytes_type ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
        == CUDA_SUCCESS;
}

template <bool NVFP4, bool GATED, int EPI>
cudaError_t launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& tp, dim3 grid,
                      cudaStream_t stream)
{
    constexpr uint32_t stage = 2 * kTileBytes + (NVFP4 ? 2 * kSfBytes : 0);
    constexpr size_t smem = kStages * stage + 1024 /* alignment slack */ + 128 /* barriers */;
    auto kernel = gemm_tc_kernel<NVFP4, GATED, EPI>;
    static bool configured[64] = {}; // per instantiation and device
    int dev = 0;
    cudaError_t derr = cudaGetDevice(&dev);
    if (derr != cudaSuccess)
        return derr;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
        if (err != cudaSuccess)
            return err;
        if (dev >= 0 && dev < 64)
            configured[dev] = true;
    }
    kernel<<<grid, kThreads, smem, stream>>>(ma, mb, tp);
    note_launch();
    return cudaGetLastError();
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

TcParams make_params(const GemmProblem& g)
{
    TcParams tp {};
    tp.n = g.n;
    tp.b_rows = g.gated ? 2 * g.n : g.n;
    tp.kgroups = g.k / 64;
    tp.k_blocks = g.nvfp4 ? (g.k + 255) / 256 : (g.k + 63) / 64;
    tp.sfa = g.a_scale_tiled;
    tp.sfb = g.b_scale_tiled;
    tp.sfb_group_stride = g.nvfp4 ? qs3_nvfp4_tiled_scale_bytes(tp.b_rows, g.k) : 0;
    tp.tile_expert = g.tile_expert;
    tp.tile_row0 = g.tile_row0;
    tp.tile_nrows = g.tile_nrows;
    tp.total_tiles = g.total_tiles;
    tp.dense_rows = static_cast<uint32_t>(g.a_rows);
    tp.out = g.out;
    tp.out_pitch = g.out_pitch_elems;
    tp.out_sf = g.out_scale_tiled;
    tp.out_kgroups = g.n / 64;
    tp.alpha = g.alpha;
    tp.beta = g.beta;
    tp.group_scale = g.group_scale;
    tp.bias = g.bias;
    tp.out_global = g.out_global_scale == 0.0f ? 1.0f : g.out_global_scale;
    tp.err = device_error_word();
    return tp;
}

} // namespace

bool gemm_tc_supported(const GemmProblem& g)
{
    if (!aligned16(g.a) || !aligned16(g.b) || g.a_pitch_bytes % 16 != 0 || g.b_pitch_bytes % 16 != 0)
        return false;
    if (g.nvfp4) {
        // scale tiles are addressed per 128 rows and per 256 k elements
        return g.k % 256 == 0 && g.n % 64 == 0 && (g.gated || g.n % 128 == 0);
    }
    return g.k % 8 == 0;
}

cudaError_t launch_gemm(const GemmProblem& g, cudaStream_t stream, const char** why)
{
    if (why != nullptr)
        *why = nullptr;
    TcParams tp = make_params(g);
    const uint32_t m_tiles = g.tile_expert != nullptr
        ? g.max_tiles
        : static_cast<uint32_t>((g.a_rows + kBM - 1) / kBM);
    if (m_tiles == 0 || g.n == 0)
        return cudaSuccess;
    if (m_tiles > 65535) {
        if (why != nullptr)
            *why = "more than 65535 row tiles";
        return cudaErrorNotSupported;
    }
    const bool force_simt = [] {
        const char* v = getenv("QS3_FORCE_SIMT");
        return v != nullptr && v[0] == '1';
    }();

    if (gemm_tc_supported(g) && !(force_simt && !g.nvfp4)) {
        const uint32_t feat = g.gated ? kBN / 2 : kBN;
        dim3 grid((g.n + feat - 1) / feat, m_tiles, 1);
        CUtensorMap ma, mb;
        const uint64_t inner = g.nvfp4 ? g.k / 2 : g.k;
        const uint64_t b_total_rows = static_cast<uint64_t>(g.groups) * tp.b_rows;
        if (!make_map(&ma, g.nvfp4, g.a, inner, g.a_rows, g.a_pitch_bytes, kBM)
            || !make_map(&mb, g.nvfp4, g.b, inner, b_total_rows, g.b_pitch_bytes, g.gated ? kBN / 2 : kBN)) {
            if (why != nullptr)
                *why = "cuTensorMapEncodeTiled failed";
            return cudaErrorInvalidValue;
        }
        if (g.nvfp4) {
            if (g.gated && g.epilogue == EPI_SWIGLU_NVFP4)
                return launch_tc<true, true, EPI_SWIGLU_NVFP4>(ma, mb, tp, grid, stream);
            if (!g.gated && g.epilogue == EPI_STORE_BF16)
                return launch_tc<true, false, EPI_STORE_BF16>(ma, mb, tp, grid, stream);
        } else {
            if (g.gated && g.epilogue == EPI_SWIGLU_BF16)
                return launch_tc<false, true, EPI_SWIGLU_BF16>(ma, mb, tp, grid, stream);
            if (!g.gated && g.epilogue == EPI_STORE_BF16)
                return launch_tc<false, false, EPI_STORE_BF16>(ma, mb, tp, grid, stream);
            if (!g.gated && g.epilogue == EPI_STORE_F32)
                return launch_tc<false, false, EPI_STORE_F32>(ma, mb, tp, grid, stream);
        }
        if (why != nullptr)
            *why = "no tensor-core kernel for this operand/epilogue combination";
        return cudaErrorNotSupported;
    }
    if (g.nvfp4) {
        if (why != nullptr)
            *why = "NVFP4 GEMM needs k % 256 == 0, n % 64 == 0 and 16-byte aligned operands";
        return cudaErrorNotSupported;
    }
    // CUDA-core kernel
    const uint32_t threads = 128;
    dim3 grid((g.n + threads - 1) / threads, m_tiles, 1);
    const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(g.a);
    const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(g.b);
    const uint64_t ap = g.a_pitch_bytes / 2, bp = g.b_pitch_bytes / 2;
    if (g.epilogue == EPI_SWIGLU_BF16)
        gemm_simt_kernel<EPI_SWIGLU_BF16><<<grid, threads, 0, stream>>>(a, ap, b, bp, tp, g.k, 1);
    else if (g.epilogue == EPI_STORE_F32)
        gemm_simt_kernel<EPI_STORE_F32><<<grid, threads, 0, stream>>>(a, ap, b, bp, tp, g.k, 0);
    else if (g.epilogue == EPI_STORE_BF16)
        gemm_simt_kernel<EPI_STORE_BF16><<<grid, threads, 0, stream>>>(a, ap, b, bp, tp, g.k, 0);
    else {
        if (why != nullptr)
            *why = "epilogue not available on the CUDA-core kernel";
        return cudaErrorNotSupported;
    }
    note_launch();
    return cudaGetLastError();
}

} // namespace qs3

extern "C" size_t qs3_nvfp4_tiled_scale_bytes(uint64_t rows, uint64_t k)
{
    return static_cast<size_t>(((rows + 127) / 128) * (k / 64) * 512);
}
