// Dense bf16 GEMM  D[m, n] = alpha * sum_k A[m, k] * B[n, k] (+ beta * D) (+ bias[n])  for the
// projection lane (qscb_gemm_bf16: router logits, shared expert in bf16 plans, LM head).
//
// The one-tile-per-CTA kernel of gemm.cu issues 128 x 128 instructions and relies on two
// co-resident CTAs to hide its epilogue. This kernel is the large-problem variant:
//
//   persistent   one CTA per SM walks the output tiles (row tile fastest, so the CTAs of a wave
//                share one or two B panels through L2)
//   128 x 256    tcgen05.mma kind::f16 with N = 256: the widest single-CTA instruction
//   TMEM         two 256-column f32 accumulators: the epilogue of tile i (eight warps, two per
//                lane quadrant) overlaps the main loop of tile i + 1
//   smem         ring of four stages, each A 128 x 64 bf16 (16 KB) + B 256 x 64 bf16 (32 KB),
//                filled by TMA with the 128-byte swizzle
//
// Rows past the end of A or B are zero-filled by TMA and masked in the epilogue. Every wait is
// bounded; on expiry the kernel records a code and leaves through the normal teardown.
#include "tcgen05.cuh"

#include <cooperative_groups.h>

#include <algorithm>

namespace qs3 {
namespace {

using namespace tc;

constexpr int kDnThreads = 320; // warps 0-7 epilogue, 8 producer, 9 MMA issuer
constexpr uint32_t kDnBN = 256;
constexpr uint32_t kDnStageBytes = 3 * kTileBytes; // A tile + two B tiles
constexpr uint32_t kDnStages = 4;
constexpr uint32_t kDnTmemCols = 512;
constexpr uint64_t kDnMinTiles = 64;

enum : uint32_t {
    ERR_DN_FULL_WAIT = 0x55000001u,
    ERR_DN_EMPTY_WAIT = 0x55000002u,
    ERR_DN_ACC_FULL_WAIT = 0x55000003u,
    ERR_DN_ACC_EMPTY_WAIT = 0x55000004u,
};

template <int EPI>
__global__ void __launch_bounds__(kDnThreads, 1)
gemm_dense_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const TcParams p, const uint32_t tiles_m, const uint32_t tiles_n)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kDnStages * kDnStageBytes);
    uint64_t* empty_bar = full_bar + kDnStages;
    uint64_t* acc_full = empty_bar + kDnStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t total = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kDnStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8); // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kDnTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ------------------------------------------------------------ producer --
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const int row0 = static_cast<int>((t % tiles_m) * kBM);
                const int col0 = static_cast<int>((t / tiles_m) * kDnBN);
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait<true>(&empty_bar[s], ph ^ 1, abort_flag, p.err, ERR_DN_EMPTY_WAIT)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + s * kDnStageBytes;
                    mbar_expect_tx(&full_bar[s], kDnStageBytes);
                    const int c0 = static_cast<int>(kb) * 64;
                    tma_load_2d(sa, &map_a, &full_bar[s], c0, row0);
                    tma_load_2d(sa + kTileBytes, &map_b, &full_bar[s], c0, col0);
                    tma_load_2d(sa + 2 * kTileBytes, &map_b, &full_bar[s], c0, col0 + 128);
                    if (++s == kDnStages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------- MMA issuer --
        if (lane == 0) {
            // M = 128, N = 256, bf16 x bf16 -> f32, both operands K-major
            constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kDnBN >> 3) << 17) | ((kBM >> 4) << 24);
            uint32_t s = 0, ph = 0, u = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x, ++u) {
                const uint32_t buf = u & 1;
                if (!mbar_wait<true>(&acc_empty[buf], ((u >> 1) & 1) ^ 1, abort_flag, p.err, ERR_DN_ACC_EMPTY_WAIT))
                    break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * kDnBN;
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait<true>(&full_bar[s], ph, abort_flag, p.err, ERR_DN_FULL_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * kDnStageBytes);
                    const uint64_t da = operand_desc(sa);
                    const uint64_t db = operand_desc(sa + kTileBytes); // 256 rows: two tiles back to back
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        tc_mma_bf16(d, da + 2 * j, db + 2 * j, kIdesc, (kb > 0 || j > 0) ? 1u : 0u);
                    tc_commit(&empty_bar[s]);
                    if (++s == kDnStages) {
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
        uint32_t u = 0;
        for (uint32_t t = blockIdx.x; t < total; t += gridDim.x, ++u) {
            const uint32_t buf = u & 1;
            const bool ready = __all_sync(
                0xffffffffu, mbar_wait(&acc_full[buf], (u >> 1) & 1, abort_flag, p.err, ERR_DN_ACC_FULL_WAIT));
            if (!ready)
                break;
            tc_fence_after();
            const int row0 = static_cast<int>((t % tiles_m) * kBM);
            const int nrows = min(kBM, static_cast<int>(p.dense_rows) - row0);
            const uint32_t nt = (t / tiles_m) * 2; // in units of the 128-column epilogue tile
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h)
                epilogue_tile<false, EPI, 2>(p, tmem_base + buf * kDnBN + h * kBN, warp & 3, lane, 0, row0, nrows,
                                             nt + h, warp >> 2);
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&acc_empty[buf]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kDnTmemCols)
                     : "memory");
    }
}

// ---- CTA-pair variant ---------------------------------------------------------------------
//
// A 128 x 256 tile needs (128 + 256) operand rows per 2 * 128 * 256 products per k: at 1.3 PFLOP/s
// that is 15 TB/s out of L2, which is what bounds the kernel above. Here two CTAs of a cluster
// (two SMs) compute one 256 x 256 tile with cta_group::2 instructions: each loads its own 128
// rows of A and HALF of the 256 B rows, the tensor cores of both SMs read both halves, and each
// CTA ends up with its 128 output rows in its own tensor memory. Operand traffic per product
// drops by a third. Every load has one destination CTA: each CTA's own TMA loads (cta_group::2
// form) signal the barrier of the pair's first CTA, which issues the MMAs for both.
//
//   barriers  full[s]      first CTA only: its expect_tx covers both CTAs' tiles of the stage
//             empty[s]     one per CTA: the first CTA commits to its own and to its peer's
//             acc_full[b]  one per CTA, same way;  acc_empty[b] first CTA only, 16 arrivals
//                          (eight epilogue warps of each CTA, the peer's through cluster addresses)
constexpr uint32_t kPrKbs = 2;                              // k blocks (of 64) per stage
constexpr uint32_t kPrStageBytes = kPrKbs * 2 * kTileBytes; // per CTA and k block: A 128 x 64, B 128 x 64
constexpr uint32_t kPrStages = 3;
constexpr uint64_t kPrMinTiles = 74;

__device__ __forceinline__ uint32_t cluster_addr(const void* local, uint32_t cta_rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(cta_rank));
    return remote;
}

// TMA tile load whose completion bytes are counted on a barrier that may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kDnThreads, 1)
gemm_dense_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const TcParams p, const uint32_t tiles_m, const uint32_t tiles_n)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = cluster.block_rank(); // 0: issues the MMAs of the pair

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPrStages * kPrStageBytes);
    uint64_t* empty_bar = full_bar + kPrStages;
    uint64_t* acc_full = empty_bar + kPrStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t total = tiles_m * tiles_n;
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kPrStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 16);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    cluster.sync(); // both CTAs resident and their barriers initialised before anything is signalled
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kDnTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster.sync();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 8) {
        // ------------------------------------------------------------ producer --
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t t = pair; t < total && ok; t += pairs) {
                const int row0 = static_cast<int>((t % tiles_m) * 256 + rank * 128);
                const int col0 = static_cast<int>((t / tiles_m) * 256 + rank * 128);
                for (uint32_t kb = 0; kb < p.k_blocks; kb += kPrKbs) {
                    if (!mbar_wait<true>(&empty_bar[s], ph ^ 1, abort_flag, p.err, ERR_DN_EMPTY_WAIT)) {
                        ok = false;
                        break;
                    }
                    const uint32_t nkb = min(kPrKbs, p.k_blocks - kb);
                    uint8_t* sa = smem + s * kPrStageBytes;
                    if (rank == 0)
                        mbar_expect_tx(&full_bar[s], nkb * 4 * kTileBytes); // both CTAs' A and B tiles
                    const uint32_t bar = cluster_addr(&full_bar[s], 0);
                    for (uint32_t q = 0; q < nkb; ++q) {
                        const int c0 = static_cast<int>(kb + q) * 64;
                        tma_load_2d_pair(sa + q * 2 * kTileBytes, &map_a, bar, c0, row0);
                        tma_load_2d_pair(sa + q * 2 * kTileBytes + kTileBytes, &map_b, bar, c0, col0);
                    }
                    if (++s == kPrStages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------- MMA issuer --
        if (rank == 0 && lane == 0) {
            // M = 256 (128 rows in each CTA), N = 256 (128 B rows from each CTA)
            constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((256u >> 4) << 24);
            uint32_t s = 0, ph = 0, u = 0;
            bool ok = true;
            for (uint32_t t = pair; t < total && ok; t += pairs, ++u) {
                const uint32_t buf = u & 1;
                if (!mbar_wait<true>(&acc_empty[buf], ((u >> 1) & 1) ^ 1, abort_flag, p.err, ERR_DN_ACC_EMPTY_WAIT))
                    break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * kDnBN;
                for (uint32_t kb = 0; kb < p.k_blocks; kb += kPrKbs) {
                    if (!mbar_wait<true>(&full_bar[s], ph, abort_flag, p.err, ERR_DN_FULL_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t nkb = min(kPrKbs, p.k_blocks - kb);
                    for (uint32_t q = 0; q < nkb; ++q) {
                        const uint32_t sa = smem_u32(smem + s * kPrStageBytes + q * 2 * kTileBytes);
                        const uint64_t da = operand_desc(sa);
                        const uint64_t db = operand_desc(sa + kTileBytes);
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            const uint32_t acc = (kb + q > 0 || j > 0) ? 1u : 0u;
                            asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %4, 0;\n\t"
                                         "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, q;\n\t}" ::"r"(d),
                                         "l"(da + 2 * j), "l"(db + 2 * j), "r"(kIdesc), "r"(acc)
                                         : "memory");
                        }
                    }
                    tc_commit_pair(cluster_addr(&empty_bar[s], 0));
                    tc_commit_pair(cluster_addr(&empty_bar[s], 1));
                    if (++s == kPrStages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) {
                    tc_commit_pair(cluster_addr(&acc_full[buf], 0));
                    tc_commit_pair(cluster_addr(&acc_full[buf], 1));
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue --
        uint32_t u = 0;
        for (uint32_t t = pair; t < total; t += pairs, ++u) {
            const uint32_t buf = u & 1;
            const bool ready = __all_sync(
                0xffffffffu, mbar_wait(&acc_full[buf], (u >> 1) & 1, abort_flag, p.err, ERR_DN_ACC_FULL_WAIT));
            if (!ready)
                break;
            tc_fence_after();
            const int row0 = static_cast<int>((t % tiles_m) * 256 + rank * 128);
            const int nrows = min(kBM, static_cast<int>(p.dense_rows) - row0);
            const uint32_t nt = (t / tiles_m) * 2;
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h)
                epilogue_tile<false, EPI, 2>(p, tmem_base + buf * kDnBN + h * kBN, warp & 3, lane, 0, row0, nrows,
                                             nt + h, warp >> 2);
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive_cluster(cluster_addr(&acc_empty[buf], 0));
        }
    }

    tc_fence_before();
    cluster.sync(); // the pair's tensor memory is idle in both CTAs
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kDnTmemCols)
                     : "memory");
    }
}

template <int EPI>
cudaError_t launch_pair_instance(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& tp, uint32_t tiles_m,
                                 uint32_t tiles_n, cudaStream_t stream)
{
    auto kernel = gemm_dense_pair_kernel<EPI>;
    constexpr size_t smem = 1024 + kPrStages * kPrStageBytes + 256;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess)
        return err;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess)
            return err;
        if (dev >= 0 && dev < 64)
            configured[dev] = true;
    }
    const uint32_t pairs = std::min(tiles_m * tiles_n, device_sm_count() / 2);
    kernel<<<2 * pairs, kDnThreads, smem, stream>>>(ma, mb, tp, tiles_m, tiles_n);
    note_launch();
    return cudaGetLastError();
}

template <int EPI>
cudaError_t launch_dense_instance(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& tp, uint32_t tiles_m,
                                  uint32_t tiles_n, cudaStream_t stream)
{
    auto kernel = gemm_dense_bf16_kernel<EPI>;
    constexpr size_t smem = 1024 + kDnStages * kDnStageBytes + 256;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess)
        return err;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess)
            return err;
        if (dev >= 0 && dev < 64)
            configured[dev] = true;
    }
    const uint32_t grid = std::min(tiles_m * tiles_n, device_sm_count());
    kernel<<<grid, kDnThreads, smem, stream>>>(ma, mb, tp, tiles_m, tiles_n);
    note_launch();
    return cudaGetLastError();
}

} // namespace

bool gemm_dense_bf16_supported(const GemmProblem& g)
{
    return !g.nvfp4 && !g.gated && g.tile_expert == nullptr && g.groups == 1 && g.a_rows > 64 && g.k % 64 == 0
        && g.k >= 64 && g.n >= 128 && (g.epilogue == EPI_STORE_BF16 || g.epilogue == EPI_STORE_F32)
        && (reinterpret_cast<uintptr_t>(g.a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(g.b) & 15u) == 0
        && g.a_pitch_bytes % 16 == 0 && g.b_pitch_bytes % 16 == 0
        && (g.a_rows + kBM - 1) / kBM * ((g.n + kDnBN - 1) / kDnBN) < (1ull << 31)
        // with fewer tiles than this the 128 x 128 kernel spreads the problem over more SMs
        && (g.a_rows + kBM - 1) / kBM * ((g.n + kDnBN - 1) / kDnBN) >= kDnMinTiles;
}

cudaError_t launch_gemm_dense_bf16(const GemmProblem& g, cudaStream_t stream, const char** why)
{
    TcParams tp {};
    tp.n = g.n;
    tp.k_blocks = g.k / 64;
    tp.b_rows = g.n;
    tp.dense_rows = static_cast<uint32_t>(g.a_rows);
    tp.out = g.out;
    tp.out_pitch = g.out_pitch_elems;
    tp.alpha = g.alpha;
    tp.beta = g.beta;
    tp.bias = g.bias;
    tp.err = device_error_word();
    const uint32_t tiles_m = static_cast<uint32_t>((g.a_rows + kBM - 1) / kBM);
    const uint32_t tiles_n = (g.n + kDnBN - 1) / kDnBN;
    CUtensorMap ma, mb;
    if (!make_operand_map(&ma, false, g.a, g.k, g.a_rows, g.a_pitch_bytes, kBM)
        || !make_operand_map(&mb, false, g.b, g.k, g.n, g.b_pitch_bytes, 128)) {
        if (why != nullptr)
            *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    // enough 256 x 256 tiles to give every CTA pair work: two SMs per tile, B shared between them
    const uint32_t pair_m = static_cast<uint32_t>((g.a_rows + 255) / 256), pair_n = (g.n + 255) / 256;
    if (static_cast<uint64_t>(pair_m) * pair_n >= kPrMinTiles && g.a_rows >= 1024)
        return g.epilogue == EPI_STORE_F32 ? launch_pair_instance<EPI_STORE_F32>(ma, mb, tp, pair_m, pair_n, stream)
                                           : launch_pair_instance<EPI_STORE_BF16>(ma, mb, tp, pair_m, pair_n, stream);
    return g.epilogue == EPI_STORE_F32 ? launch_dense_instance<EPI_STORE_F32>(ma, mb, tp, tiles_m, tiles_n, stream)
                                       : launch_dense_instance<EPI_STORE_BF16>(ma, mb, tp, tiles_m, tiles_n, stream);
}

} // namespace qs3
