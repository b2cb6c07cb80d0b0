// tcgen05 / TMA / mbarrier PTX wrappers, descriptor builders and the fused epilogue
// shared by the tensor-core GEMM kernels of this library (sm_100a only).
#pragma once

#include "common.cuh"
#include "nvfp4.cuh"

namespace qs3 {
namespace tc {

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
    const float* group_scale_up; // gated tiles: multiplier of the up columns (NULL: group_scale)
    const float* bias;
    float out_global;
    uint32_t* err;
    uint32_t tma_store; // resident-A kernel, bf16 output: stage the tile in smem and store it with TMA
    // split-k launches of gemm_tc_kernel (grid.z slices): slice z reduces k blocks [z * split_kb, +split_kb)
    // and writes its partial tile split_row_stride * z rows further down the output; 0: no split
    uint32_t split_kb;
    uint32_t split_row_stride;
};

// Host helpers defined beside the GEMM launchers. make_operand_map: 2-D tensor map over a
// row-major [rows, inner] operand (bf16 elements, or bytes when `bytes_type`), box =
// 128 bytes x box_rows with the 128-byte swizzle.
} // namespace tc
bool make_operand_map(CUtensorMap* map, bool bytes_type, const void* base, uint64_t inner_elems, uint64_t rows,
                      uint64_t pitch_bytes, uint32_t box_rows);
uint32_t device_sm_count();
namespace tc {

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

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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

__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}

// Bounded wait; on expiry records `code` and raises the CTA's abort flag. POLL selects
// non-blocking test_wait polling (lowest wake-up latency; for the single producer and
// MMA threads) instead of the suspending try_wait (for whole epilogue warps).
template <bool POLL = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* err, uint32_t code, uint64_t limit_cycles = kWaitCycles)
{
    if (POLL ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity))
        return true;
    const uint64_t start = clock64();
    uint32_t spins = 0;
    while (true) {
        if (POLL ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity))
            return true;
        if (POLL && (++spins & 63u) != 0)
            continue;
        if (*abort_flag != 0)
            return false;
        if (static_cast<uint64_t>(clock64()) - start > limit_cycles) {
            *abort_flag = 1;
            if (err != nullptr)
                atomicCAS(err, 0u, code);
            return false;
        }
    }
}

// AND of `pred` over the `nthreads` threads that meet at named barrier `bar_id`, returned to all of
// them. Epilogue warps that synchronise with each other per tile take their "stop, a wait gave up"
// decision through this, so that no warp is left waiting at a barrier the others walked away from.
__device__ __forceinline__ bool group_all(uint32_t bar_id, uint32_t nthreads, bool pred)
{
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %3, 0;\n\t"
                 "bar.red.and.pred p, %1, %2, q;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(r)
                 : "r"(bar_id), "r"(nthreads), "r"(static_cast<uint32_t>(pred))
                 : "memory");
    return r != 0;
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

// e4m3 x e4m3 (formats are in the instruction descriptor), K = 32 elements per instruction
__device__ __forceinline__ void tc_mma_f8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
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

// Fused epilogue of one 128-row accumulator tile whose first TMEM column is `tmem_acc`:
// plain tiles hold kBN output columns, gated tiles kBN/2 gate columns followed by their
// kBN/2 up columns. Must be called by whole warps (tcgen05.ld is warp-collective);
// `warp` is the TMEM lane quadrant 0..3 the calling warp may read. With HALVES == 2 two
// warps share a quadrant and `half` (0 / 1) selects which half of the column chunks
// this warp handles.
template <bool GATED, int EPI, int HALVES = 1>
__device__ __forceinline__ void epilogue_tile(const TcParams& p, uint32_t tmem_acc, uint32_t warp, uint32_t lane,
                                              int expert, int row0, int nrows, uint32_t nt, uint32_t half = 0)
{
    constexpr uint32_t kFeat = GATED ? kBN / 2 : kBN;
    const uint32_t n0 = nt * kFeat;
    const uint32_t tmem_base = tmem_acc;
    const int r = static_cast<int>(warp * 32 + lane); // tile row = TMEM lane
    const bool row_ok = r < nrows;
    const uint64_t grow = static_cast<uint64_t>(row0) + r;
    const uint32_t lane_base = (warp * 32) << 16;
    float scale = p.alpha == 0.0f ? 1.0f : p.alpha;
    float scale_up = scale; // gate and up rows of an expert may carry different global scales
    if (p.group_scale != nullptr)
        scale *= p.group_scale[expert];
    scale_up *= p.group_scale_up != nullptr ? p.group_scale_up[expert]
                                            : (p.group_scale != nullptr ? p.group_scale[expert] : 1.0f);

    if constexpr (!GATED) {
        constexpr uint32_t kChunks = kBN / 16 / HALVES;
        for (uint32_t c = half * kChunks; c < (half + 1) * kChunks; ++c) {
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
        constexpr uint32_t kChunks = kFeat / 16 / HALVES;
        for (uint32_t c = half * kChunks; c < (half + 1) * kChunks; ++c) {
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
                    const float u = round_bf16(__uint_as_float(vu[i]) * scale_up);
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
                    const float u = __uint_as_float(vu[i]) * scale_up;
                    act[i] = __fdividef(g, 1.0f + __expf(-g)) * u;
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
            if (row_ok && n0 < p.n) {
                uint8_t* dst = p.out_sf + tiled_scale_offset(grow, 4ull * nt, p.out_kgroups);
                if constexpr (HALVES == 1)
                    *reinterpret_cast<uint32_t*>(dst) = sf_word;
                else
                    *reinterpret_cast<uint16_t*>(dst + 2 * half) = static_cast<uint16_t>(sf_word >> (16 * half));
            }
        }
    }
}

} // namespace tc
} // namespace qs3
