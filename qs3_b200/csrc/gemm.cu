// Grouped / dense GEMM  D[m, n] = sum_k A[m, k] * B[g][n, k]. Kernels in this file:
//   gemm_tc_kernel        tcgen05, one 128 x 128 tile per CTA: grouped bf16 problems, NVFP4 with k > 2048
//                         (dense bf16 problems with more than 64 rows go to gemm_dense.cu)
//   gemm_tc_astat_kernel  tcgen05, NVFP4 with the A panel resident in shared memory (k <= 2048)
//   gemm_skinny_kernel    CUDA cores, bf16 with at most 64 rows (router logits of a decode batch)
//   gemm_simt_kernel      CUDA cores, shapes the tensor-core tiles cannot address
// launch_gemm() at the end picks one of these, the dense kernel of gemm_dense.cu or the decode
// kernel of nvfp4_decode.cu.
//
// gemm_tc_kernel: one 128 x 128 output tile per CTA on the 5th-generation tensor cores:
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
#include "tcgen05.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>

namespace qs3 {

namespace {

using namespace tc;

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
    // the k blocks this CTA reduces (all of them unless the launch is split over grid.z)
    const uint32_t kb_base = p.split_kb != 0 ? blockIdx.z * p.split_kb : 0u;
    const uint32_t kb_count = p.split_kb != 0 ? min(p.split_kb, p.k_blocks - kb_base) : p.k_blocks;

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
            for (uint32_t kb = 0; kb < kb_count; ++kb) {
                const uint32_t s = kb % kStages;
                const uint32_t ph = (kb / kStages) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.err, ERR_EMPTY_WAIT))
                    break;
                uint8_t* sa = smem + s * kStageBytes;
                uint8_t* sb = sa + kTileBytes;
                mbar_expect_tx(&full_bar[s], kStageBytes);
                // inner coordinate in elements of the map's type (bf16 elements / bytes)
                const int c0 = static_cast<int>(kb_base + kb) * (NVFP4 ? 128 : 64);
                tma_load_2d(sa, &map_a, &full_bar[s], c0, row0);
                if (GATED) {
                    tma_load_2d(sb, &map_b, &full_bar[s], c0, b_row);
                    tma_load_2d(sb + kTileBytes / 2, &map_b, &full_bar[s], c0,
                                b_row + static_cast<int>(p.n));
                } else {
                    tma_load_2d(sb, &map_b, &full_bar[s], c0, b_row);
                }
                if (NVFP4) {
                    bulk_load(sb + kTileBytes, sfa_src + static_cast<uint64_t>(kb_base + kb) * kSfBytes, kSfBytes,
                              &full_bar[s]);
                    bulk_load(sb + kTileBytes + kSfBytes, sfb_src + static_cast<uint64_t>(kb_base + kb) * kSfBytes,
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
            for (uint32_t kb = 0; kb < kb_count; ++kb) {
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
            epilogue_tile<GATED, EPI>(p, tmem_base, warp, lane, expert,
                                      row0 + static_cast<int>(blockIdx.z * p.split_row_stride), nrows, nt);
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

// ---- NVFP4 kernel with a resident A panel ------------------------------------------------
//
// The 128 x 128 kernel above re-streams its A tile for every column tile, so each byte
// brought into shared memory feeds only ~233 FLOP and the kernel is bound by L2 -> SM
// operand delivery. Here one CTA owns a 128-row tile, loads the whole [128, k] A panel
// (codes: k/2 bytes per row, up to 128 KB; scales: straight into tensor memory) ONCE and
// then walks its share of the column tiles streaming only B through the ring, which
// doubles the FLOP per streamed byte. Two 128-column accumulators in tensor memory
// alternate, so the epilogue of column tile i overlaps the MMAs of tile i + 1.
//
//   TMEM: [0,128) acc 0 | [128,256) acc 1 | [256,384) A scales (k/64 * 4 columns) | [384,512) B scales
//         (16 columns per k block of every ring stage)
//
// The scale copies into tensor memory (tcgen05.cp) are issued by a warp of their own: as part of
// the MMA thread's instruction stream each one stalls the tensor pipe for ~50 cycles (four of them
// per k block cost as much as two of its four MMAs), from another thread they cost nothing. The
// copier hands a stage's scales to the MMA thread through an mbarrier (tcgen05.commit); the scale
// columns of a ring stage are free again when the stage itself has been refilled.
//   smem: A panel k_blocks x 16 KB | A-scale staging k_blocks x 2 KB | ring of stages, each one or
//         two k blocks of (16 KB B + 2 KB scales) | bf16 output: two 32 KB staging tiles
//
// Epilogue, eight warps: with the SwiGLU / f32 / plain-store epilogues two warps share a
// TMEM lane quadrant and split the columns of one tile; with bf16 tiles written through TMA
// stores the warps form two groups that take alternate column tiles.
//
// Grid: (n_splits, row tiles). A CTA handles column tiles [split * per, ...); n_splits > 1
// only when there are too few row tiles to fill the GPU.
constexpr int kAsMaxKBlocks = 8;   // k <= 2048
constexpr int kAsMaxStages = 8;
constexpr uint32_t kSmallTileRows = 32; // bf16-output tiles with at most this many rows store them directly
constexpr int kAsThreads = 352;    // warps 0-7 epilogue (two per TMEM lane quadrant), 8 producer, 9 MMA, 10 scale copier
constexpr uint32_t kAsStageBytes = kTileBytes + kSfBytes;

enum : uint32_t {
    ERR_AS_PANEL_WAIT = 0x52000001u,
    ERR_AS_FULL_WAIT = 0x52000002u,
    ERR_AS_EMPTY_WAIT = 0x52000003u,
    ERR_AS_ACC_FULL_WAIT = 0x52000004u,
    ERR_AS_ACC_EMPTY_WAIT = 0x52000005u,
    ERR_AS_SF_WAIT = 0x52000006u,
};

template <bool GATED, int EPI>
__global__ void __launch_bounds__(kAsThreads, 1)
gemm_tc_astat_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_o, const TcParams p, const uint32_t stages,
                     const uint32_t nt_per_split, const uint32_t kbs)
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
    constexpr uint32_t kFeat = GATED ? kBN / 2 : kBN;
    const uint32_t n_tiles = (p.n + kFeat - 1) / kFeat;
    const uint32_t nt_begin = blockIdx.x * nt_per_split;
    const uint32_t nt_end = min(n_tiles, nt_begin + nt_per_split);
    if (nt_begin >= nt_end)
        return;
    const uint32_t kb_count = p.k_blocks;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* a_panel = smem;
    uint8_t* sfa_stage = a_panel + kb_count * kTileBytes;
    uint8_t* ring = sfa_stage + kb_count * kSfBytes;
    uint8_t* staging = ring + stages * kbs * kAsStageBytes; // two 32 KB output tiles, only with p.tma_store
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + (p.tma_store ? 4 * kTileBytes : 0));
    uint64_t* empty_bar = full_bar + kAsMaxStages;
    uint64_t* acc_full = empty_bar + kAsMaxStages;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* panel_bar = acc_empty + 2;
    uint64_t* sfa_ready = panel_bar + 1;
    uint64_t* sf_ready = sfa_ready + 1;            // [kAsMaxStages]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_ready + kAsMaxStages);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    constexpr uint32_t kTmemCols = 512;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
            mbar_init(&sf_ready[s], 1);
        }
        mbar_init(sfa_ready, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            // one arrival per epilogue warp that reads the buffer (a group of four with TMA stores)
            mbar_init(&acc_empty[b], (EPI == EPI_STORE_BF16 && p.tma_store) ? 4 : 8);
        }
        mbar_init(panel_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sfa = tmem_base + 256;
    const uint32_t tmem_sfb = tmem_base + 384; // 16 columns per k block of every ring stage
    const uint32_t stage_bytes = kbs * kAsStageBytes;   // kbs k-blocks of B codes, then their scales
    const uint32_t stages_per_tile = kb_count / kbs;

    if (warp == 8) {
        // ------------------------------------------------------------ producer --
        if (lane == 0) {
            // the A panel and its scales, once
            mbar_expect_tx(panel_bar, kb_count * (kTileBytes + kSfBytes));
            for (uint32_t kb = 0; kb < kb_count; ++kb)
                tma_load_2d(a_panel + kb * kTileBytes, &map_a, panel_bar, static_cast<int>(kb) * 128, row0);
            bulk_load(sfa_stage, p.sfa + (static_cast<uint64_t>(row0 >> 7) * p.kgroups) * 512,
                      kb_count * kSfBytes, panel_bar);
            // B tiles of every column tile of this CTA
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t nt = nt_begin; ok && nt < nt_end; ++nt) {
                const int b_row = expert * static_cast<int>(p.b_rows) + static_cast<int>(nt * kFeat);
                const uint8_t* sfb_src = p.sfb + static_cast<uint64_t>(expert) * p.sfb_group_stride
                    + (static_cast<uint64_t>(nt) * p.kgroups) * 512;
                for (uint32_t st = 0; st < stages_per_tile; ++st) {
                    if (!mbar_wait<true>(&empty_bar[s], ph ^ 1, abort_flag, p.err, ERR_AS_EMPTY_WAIT)) {
                        ok = false;
                        break;
                    }
                    uint8_t* sb = ring + s * stage_bytes;
                    mbar_expect_tx(&full_bar[s], stage_bytes);
                    for (uint32_t q = 0; q < kbs; ++q) {
                        const int c0 = static_cast<int>(st * kbs + q) * 128;
                        uint8_t* dst = sb + q * kTileBytes;
                        if (GATED) {
                            tma_load_2d(dst, &map_b, &full_bar[s], c0, b_row);
                            tma_load_2d(dst + kTileBytes / 2, &map_b, &full_bar[s], c0,
                                        b_row + static_cast<int>(p.n));
                        } else {
                            tma_load_2d(dst, &map_b, &full_bar[s], c0, b_row);
                        }
                    }
                    bulk_load(sb + kbs * kTileBytes, sfb_src + static_cast<uint64_t>(st * kbs) * kSfBytes,
                              kbs * kSfBytes, &full_bar[s]);
                    if (++s == stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------- MMA issuer --
        if (lane == 0) {
            constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24);
            // the copier has put the A scales into tensor memory (which also means the A panel has landed)
            bool ok = mbar_wait<true>(sfa_ready, 0, abort_flag, p.err, ERR_AS_PANEL_WAIT);
            const uint32_t a_addr = smem_u32(a_panel);
            uint32_t s = 0, ph = 0;
            for (uint32_t nt = nt_begin; ok && nt < nt_end; ++nt) {
                const uint32_t local = nt - nt_begin;
                const uint32_t buf = local & 1;
                const uint32_t use = local >> 1;
                if (!mbar_wait<true>(&acc_empty[buf], (use & 1) ^ 1, abort_flag, p.err, ERR_AS_ACC_EMPTY_WAIT)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + buf * kBN;
                for (uint32_t st = 0; st < stages_per_tile; ++st) {
                    // the stage's B scales are in tensor memory (the copier waited for the stage's loads)
                    if (!mbar_wait<true>(&sf_ready[s], ph, abort_flag, p.err, ERR_AS_SF_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sb = smem_u32(ring + s * stage_bytes);
                    for (uint32_t q = 0; q < kbs; ++q) {
                        const uint32_t kb = st * kbs + q;
                        const uint32_t sfb_cols = tmem_sfb + 16 * (s * kbs + q);
                        const uint64_t da = operand_desc(a_addr + kb * kTileBytes);
                        const uint64_t db = operand_desc(sb + q * kTileBytes);
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j)
                            tc_mma_nvfp4(tmem_acc, da + 2 * j, db + 2 * j, kIdesc, (kb > 0 || j > 0) ? 1u : 0u,
                                         tmem_sfa + 16 * kb + 4 * j, sfb_cols + 4 * j);
                    }
                    tc_commit(&empty_bar[s]);
                    if (++s == stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok)
                    tc_commit(&acc_full[buf]);
            }
        }
    } else if (warp == 10) {
        // -------------------------------------------------------- scale copier --
        if (lane == 0) {
            bool ok = mbar_wait<true>(panel_bar, 0, abort_flag, p.err, ERR_AS_PANEL_WAIT);
            if (ok) {
                tc_fence_after();
                // A scales: one 512-byte tile per 64 k elements -> 4 TMEM columns each
                for (uint32_t g = 0; g < kb_count * 4; ++g)
                    tc_cp_scales(tmem_sfa + 4 * g, scale_desc(smem_u32(sfa_stage) + g * 512));
                tc_commit(sfa_ready);
            }
            uint32_t s = 0, ph = 0;
            for (uint32_t nt = nt_begin; ok && nt < nt_end; ++nt) {
                for (uint32_t st = 0; st < stages_per_tile; ++st) {
                    // the stage was refilled, so the MMAs that read its scale columns last time round are done
                    if (!mbar_wait<true>(&full_bar[s], ph, abort_flag, p.err, ERR_AS_FULL_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sf_smem = smem_u32(ring + s * stage_bytes) + kbs * kTileBytes;
                    for (uint32_t q = 0; q < kbs; ++q) {
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j)
                            tc_cp_scales(tmem_sfb + 16 * (s * kbs + q) + 4 * j, scale_desc(sf_smem + q * kSfBytes + j * 512));
                    }
                    tc_commit(&sf_ready[s]);
                    if (++s == stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (EPI == EPI_STORE_BF16 && p.tma_store) {
        // ------------------------------------- epilogue, bf16 tiles through TMA stores --
        // Two groups of four warps; group g owns accumulator g and staging tile g and takes
        // every second column tile, so two tiles are in flight in the epilogue: the chain
        // wait -> tcgen05.ld -> convert -> shared memory -> TMA store of one tile is longer
        // than the MMAs of a tile with a short k. Every row of the tile is written: rows past
        // the segment end are padding rows of the same expert, rows past the tensor are clipped.
        // Tiles of at most kSmallTileRows rows skip the staging and store their rows directly.
        const uint32_t group = warp >> 2, quad = warp & 3;
        const uint32_t r = quad * 32 + lane;
        const bool issuer = quad == 0 && lane == 0;
        uint8_t* stage_buf = staging + group * 2 * kTileBytes;
        const bool small_tile = nrows <= static_cast<int>(kSmallTileRows);
        float scale = p.alpha == 0.0f ? 1.0f : p.alpha;
        if (p.group_scale != nullptr)
            scale *= p.group_scale[expert];
        for (uint32_t nt = nt_begin + group; nt < nt_end; nt += 2) {
            const uint32_t use = (nt - nt_begin) >> 1;
            bool ready = __all_sync(
                0xffffffffu, mbar_wait(&acc_full[group], use & 1, abort_flag, p.err, ERR_AS_ACC_FULL_WAIT));
            if (!small_tile)
                ready = group_all(1 + group, 128, ready); // the group meets at its barrier below: stop together
            if (!ready)
                break;
            tc_fence_after();
            if (small_tile) {
                // a tile with few rows (an expert that got a handful of tokens): only the warps that
                // own valid rows read the accumulator, and they store those rows directly
                if (quad * 32 < static_cast<uint32_t>(nrows))
                    epilogue_tile<false, EPI_STORE_BF16, 1>(p, tmem_base + group * kBN, quad, lane, expert, row0,
                                                            nrows, nt);
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&acc_empty[group]);
                continue;
            }
            if (issuer) // this group's previous store must have left the staging tile
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            asm volatile("bar.sync %0, 128;" ::"r"(1 + group) : "memory");
#pragma unroll
            for (uint32_t h2 = 0; h2 < 2; ++h2) {
                uint32_t v[4][16];
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c)
                    tc_ld16(tmem_base + group * kBN + ((quad * 32) << 16) + h2 * 64 + c * 16, v[c]);
                tc_ld_wait();
                uint8_t* row_smem = stage_buf + h2 * kTileBytes + r * 128;
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) {
                    uint32_t w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        w[i] = pack_bf16x2(__uint_as_float(v[c][2 * i]) * scale,
                                           __uint_as_float(v[c][2 * i + 1]) * scale);
                    *reinterpret_cast<uint4*>(row_smem + (((2 * c) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(row_smem + (((2 * c + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
            // the accumulator is free again; publish the staged tile to the async proxy
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&acc_empty[group]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync %0, 128;" ::"r"(1 + group) : "memory");
            if (issuer) {
                const int n0 = static_cast<int>(nt * kBN);
                for (int h2 = 0; h2 < 2; ++h2) {
                    if (n0 + h2 * 64 < static_cast<int>(p.n))
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                         reinterpret_cast<uint64_t>(&map_o)),
                                     "r"(smem_u32(stage_buf + h2 * kTileBytes)), "r"(n0 + h2 * 64), "r"(row0)
                                     : "memory");
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
        if (issuer)
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); // stores done before smem goes away
    } else {
        // ------------------------------------------------------------ epilogue --
        for (uint32_t nt = nt_begin; nt < nt_end; ++nt) {
            const uint32_t local = nt - nt_begin;
            const uint32_t buf = local & 1;
            const uint32_t use = local >> 1;
            const bool ready = __all_sync(
                0xffffffffu, mbar_wait(&acc_full[buf], use & 1, abort_flag, p.err, ERR_AS_ACC_FULL_WAIT));
            if (!ready)
                break;
            tc_fence_after();
            epilogue_tile<GATED, EPI, 2>(p, tmem_base + buf * kBN, warp & 3, lane, expert, row0, nrows, nt,
                                             warp >> 2);
            // hand the accumulator back once every lane of the warp has read it
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
    float scale_up = scale;
    if (p.group_scale != nullptr)
        scale *= p.group_scale[expert];
    scale_up *= p.group_scale_up != nullptr ? p.group_scale_up[expert]
                                            : (p.group_scale != nullptr ? p.group_scale[expert] : 1.0f);
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
            const float u = round_bf16(acc2 * scale_up);
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

template <bool GATED, int EPI>
cudaError_t launch_astat(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const TcParams& tp,
                         dim3 grid, uint32_t nt_per_split, cudaStream_t stream)
{
    constexpr size_t kSmemBudget = 227 * 1024 - 1024 /* alignment slack */ - 512 /* barriers */;
    const size_t panel = static_cast<size_t>(tp.k_blocks) * (kTileBytes + kSfBytes);
    // two k-blocks per ring stage: one barrier round trip of the single issuing thread
    // costs about as much as four 128x128x64 MMAs, so stages carry eight of them
    const uint32_t kbs = tp.k_blocks % 2 == 0 ? 2u : 1u;
    const size_t staging = tp.tma_store ? 4 * kTileBytes : 0;
    uint32_t stages = static_cast<uint32_t>((kSmemBudget - panel - staging) / (kbs * kAsStageBytes));
    stages = std::min<uint32_t>(stages, kAsMaxStages / kbs); // 16 scale columns per k block in flight, 128 in all
    const size_t smem = panel + staging + static_cast<size_t>(stages) * kbs * kAsStageBytes + 1024 + 512;
    auto kernel = gemm_tc_astat_kernel<GATED, EPI>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess)
        return err;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (err != cudaSuccess)
            return err;
        if (dev >= 0 && dev < 64)
            configured[dev] = true;
    }
    kernel<<<grid, kAsThreads, smem, stream>>>(ma, mb, mo, tp, stages, nt_per_split, kbs);
    note_launch();
    return cudaGetLastError();
}

uint32_t sm_count()
{
    static int count[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return 148;
    if (count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        count[dev] = n;
    }
    return static_cast<uint32_t>(count[dev]);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool pair_down_enabled()
{
    static const bool enabled = [] {
        const char* v = std::getenv("QS3_NVFP4_PAIR_DOWN");
        return v != nullptr && v[0] == '1';
    }();
    return enabled;
}

// ---- skinny bf16 GEMM for decode-sized batches ------------------------------------------------
//
// out[t, n] = sum_k A[t, k] * B[n, k] for a handful of rows (router logits of a decode batch):
// one 128 x 128 tensor-core tile would stream all of k through a single SM, so instead every
// output feature gets a block; a warp keeps its slice of the weight row in registers and
// walks two rows of A (L2-resident), lanes split k, one shuffle reduction per output.
constexpr uint32_t kSkinnyWarps = 8;
constexpr uint32_t kSkinnyRowsPerWarp = 2;
constexpr uint32_t kSkinnyMaxChunks = 16; // k <= 4096, in 256-element chunks (8 per lane)

__global__ void __launch_bounds__(kSkinnyWarps * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ a, uint64_t a_pitch, const __nv_bfloat16* __restrict__ b,
                   uint64_t b_pitch, uint32_t rows, uint32_t k, float* __restrict__ out, uint64_t out_pitch,
                   float alpha, float beta, const float* __restrict__ bias)
{
    const uint32_t n = blockIdx.x;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t chunks = k / 256;
    const uint4* wrow = reinterpret_cast<const uint4*>(b + static_cast<uint64_t>(n) * b_pitch);
    uint4 wv[kSkinnyMaxChunks];
#pragma unroll
    for (uint32_t c = 0; c < kSkinnyMaxChunks; ++c)
        wv[c] = c < chunks ? wrow[c * 32 + lane] : make_uint4(0, 0, 0, 0);
    const uint32_t row0 = (blockIdx.y * kSkinnyWarps + warp) * kSkinnyRowsPerWarp;
    for (uint32_t r = row0; r < min(rows, row0 + kSkinnyRowsPerWarp); ++r) {
        const uint4* xrow = reinterpret_cast<const uint4*>(a + static_cast<uint64_t>(r) * a_pitch);
        float acc = 0.0f;
#pragma unroll
        for (uint32_t c = 0; c < kSkinnyMaxChunks; ++c) {
            if (c < chunks) {
                const uint4 xv = xrow[c * 32 + lane];
                const uint32_t xs[4] = { xv.x, xv.y, xv.z, xv.w };
                const uint32_t ws[4] = { wv[c].x, wv[c].y, wv[c].z, wv[c].w };
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc = fmaf(bf16_bits_to_f32(xs[j] & 0xffffu), bf16_bits_to_f32(ws[j] & 0xffffu), acc);
                    acc = fmaf(bf16_bits_to_f32(xs[j] >> 16), bf16_bits_to_f32(ws[j] >> 16), acc);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) {
            float* o = out + static_cast<uint64_t>(r) * out_pitch + n;
            float v = acc * (alpha == 0.0f ? 1.0f : alpha);
            if (beta != 0.0f)
                v += beta * *o;
            if (bias != nullptr)
                v += bias[n];
            *o = v;
        }
    }
}

// out[r, n] = alpha * sum over slices (in slice order) of partial[slice][r, n] + beta * out[r, n] + bias[n];
// four features per thread. `partial` is [slices][rows_pad, n] f32, slice_stride elements apart.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, uint32_t slices, uint64_t slice_stride, uint64_t rows,
                     uint32_t n, float* __restrict__ out, uint64_t out_pitch, float alpha, float beta,
                     const float* __restrict__ bias)
{
    const uint64_t q = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint32_t per_row = n / 4;
    if (q >= rows * per_row)
        return;
    const uint64_t r = q / per_row;
    const uint32_t c = static_cast<uint32_t>(q % per_row) * 4;
    float4 acc = *reinterpret_cast<const float4*>(partial + r * n + c);
    for (uint32_t s = 1; s < slices; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(partial + s * slice_stride + r * n + c);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
    }
    float* o = out + r * out_pitch + c;
    float f[4] = { acc.x * alpha, acc.y * alpha, acc.z * alpha, acc.w * alpha };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (beta != 0.0f)
            f[i] += beta * o[i];
        if (bias != nullptr)
            f[i] += bias[c + i];
        o[i] = f[i];
    }
}

// Dense bf16 problem with f32 output whose rows would not fill one tensor-core tile.
bool skinny_supported(const GemmProblem& g)
{
    return !g.nvfp4 && !g.gated && g.epilogue == EPI_STORE_F32 && g.tile_expert == nullptr && g.groups == 1
        && g.group_scale == nullptr && g.a_rows <= 64 && g.k % 256 == 0 && g.k / 256 <= kSkinnyMaxChunks
        && aligned16(g.a) && aligned16(g.b) && g.a_pitch_bytes % 16 == 0 && g.b_pitch_bytes % 16 == 0
        && g.n <= 65535;
}

cudaError_t launch_skinny(const GemmProblem& g, cudaStream_t stream)
{
    const uint32_t rows = static_cast<uint32_t>(g.a_rows);
    const dim3 grid(g.n, (rows + kSkinnyWarps * kSkinnyRowsPerWarp - 1) / (kSkinnyWarps * kSkinnyRowsPerWarp));
    gemm_skinny_kernel<<<grid, kSkinnyWarps * 32, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(g.a), g.a_pitch_bytes / 2, static_cast<const __nv_bfloat16*>(g.b),
        g.b_pitch_bytes / 2, rows, g.k, static_cast<float*>(g.out), g.out_pitch_elems, g.alpha, g.beta, g.bias);
    note_launch();
    return cudaGetLastError();
}

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
    tp.group_scale_up = g.group_scale_up;
    tp.bias = g.bias;
    tp.out_global = g.out_global_scale == 0.0f ? 1.0f : g.out_global_scale;
    tp.err = device_error_word();
    return tp;
}

} // namespace

bool make_operand_map(CUtensorMap* map, bool bytes_type, const void* base, uint64_t inner_elems, uint64_t rows,
                      uint64_t pitch_bytes, uint32_t box_rows)
{
    return make_map(map, bytes_type, base, inner_elems, rows, pitch_bytes, box_rows);
}

uint32_t device_sm_count() { return sm_count(); }

bool make_scale_tile_map(CUtensorMap* map, const void* base, uint64_t tiles, uint32_t box_tiles)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr || tiles == 0 || box_tiles == 0 || box_tiles > 256)
        return false;
    const cuuint64_t dims[2] = { 128, tiles };          // 128 x u32 = one 512-byte tile per row
    const cuuint64_t strides[1] = { 512 };
    const cuuint32_t box[2] = { 128, box_tiles };
    const cuuint32_t estr[2] = { 1, 1 };
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
        == CUDA_SUCCESS;
}

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

bool make_scale_block_map(CUtensorMap* map, const void* base, uint64_t row_blocks, uint32_t kgroups,
                          uint32_t box_blocks)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr || row_blocks == 0 || kgroups < 4)
        return false;
    const cuuint64_t dims[3] = { 128, kgroups, row_blocks };
    const cuuint64_t strides[2] = { 512, static_cast<cuuint64_t>(kgroups) * 512 };
    const cuuint32_t box[3] = { 128, 4, box_blocks };
    const cuuint32_t estr[3] = { 1, 1, 1 };
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
        == CUDA_SUCCESS;
}

bool make_gated_weight_map(CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t inter,
                           uint64_t groups, uint64_t pitch_bytes, uint32_t box_halves)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr || inter < 64 || groups == 0)
        return false;
    const cuuint64_t dims[3] = { inner_bytes, inter, 2 * groups };
    const cuuint64_t strides[2] = { pitch_bytes, inter * pitch_bytes };
    const cuuint32_t box[3] = { 128, 64, box_halves };
    const cuuint32_t estr[3] = { 1, 1, 1 };
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
        == CUDA_SUCCESS;
}

// CTA-pair kernel: grouped problems with pair tiles from the route sort, and dense problems with
// enough 256-row tiles to be worth pairing. QS3_NVFP4_PAIR=0 in the environment keeps the
// single-CTA kernels (for A/B measurements).
static bool pair_kernel_wanted(const GemmProblem& g)
{
    static const bool enabled = [] {
        const char* v = std::getenv("QS3_NVFP4_PAIR");
        return v == nullptr || v[0] != '0';
    }();
    if (!enabled || !nvfp4_pair_gemm_supported(g))
        return false;
    if (g.tile_expert != nullptr)
        return g.gated != 0 || pair_down_enabled();
    return g.a_rows >= 1024 && (g.gated != 0 || pair_down_enabled());
}

cudaError_t launch_gemm(const GemmProblem& g, cudaStream_t stream, const char** why)
{
    if (why != nullptr)
        *why = nullptr;
    if (g.nvfp4 && g.tile_expert != nullptr && g.tile_rows != 0 && g.tile_rows != static_cast<uint32_t>(kBM))
        return launch_nvfp4_swap_gemm(g, stream, why);
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
    if (skinny_supported(g))
        return launch_skinny(g, stream);
    if (gemm_dense_bf16_supported(g))
        return launch_gemm_dense_bf16(g, stream, why);
    if (pair_kernel_wanted(g))
        return launch_nvfp4_pair_gemm(g, stream, why);
    if (gemm_tc_supported(g)) {
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
        if (g.nvfp4 && tp.k_blocks <= kAsMaxKBlocks) {
            // resident-A kernel: row tiles (estimated on the host) decide how far the
            // column tiles of one row tile are split over CTAs
            const uint32_t n_tiles = grid.x;
            const uint32_t m_est = g.tile_expert != nullptr
                ? (g.max_tiles > g.groups ? g.max_tiles - g.groups : 1u)
                : m_tiles;
            const uint32_t want_splits = std::max(1u, (2u * sm_count() + m_est - 1) / m_est);
            const uint32_t nt_per = std::max(1u, (n_tiles + want_splits - 1) / want_splits);
            const uint32_t splits = (n_tiles + nt_per - 1) / nt_per;
            dim3 agrid(splits, m_tiles, 1);
            if (g.gated && g.epilogue == EPI_SWIGLU_NVFP4)
                return launch_astat<true, EPI_SWIGLU_NVFP4>(ma, mb, ma, tp, agrid, nt_per, stream);
            if (!g.gated && g.epilogue == EPI_STORE_BF16) {
                // bf16 output through shared memory + TMA store when the output is a plain
                // row-major matrix whose rows may all be written (no beta read-modify-write)
                CUtensorMap mo = ma;
                TcParams tpo = tp;
                if (g.beta == 0.0f && aligned16(g.out) && (g.out_pitch_elems * 2) % 16 == 0
                    && make_map(&mo, false, g.out, g.n, g.a_rows, g.out_pitch_elems * 2, kBM))
                    tpo.tma_store = 1;
                return launch_astat<false, EPI_STORE_BF16>(ma, mb, mo, tpo, agrid, nt_per, stream);
            }
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
            if (!g.gated && g.epilogue == EPI_STORE_F32) {
                // A handful of output tiles with a long k (router logits of a decode batch: 128 x 512 x 2048
                // = four tiles) would stream all of k through four SMs: split k over grid.z, partial tiles
                // into the caller's scratch, then one pass that sums the slices in slice order (so the
                // result does not depend on timing) and applies alpha, beta and the bias.
                const uint32_t tiles = grid.x * grid.y;
                uint32_t splits = 1;
                if (g.splitk_scratch != nullptr && g.tile_expert == nullptr && 8 * tiles <= sm_count()
                    && tp.k_blocks >= 8) {
                    splits = std::min<uint32_t>({ 8u, tp.k_blocks / 4, sm_count() / tiles });
                    const size_t need = static_cast<size_t>(splits) * grid.y * kBM * g.n * sizeof(float);
                    if (splits < 2 || need > g.splitk_scratch_bytes || !aligned16(g.splitk_scratch) || g.n % 4 != 0)
                        splits = 1;
                }
                if (splits > 1) {
                    TcParams ts = tp;
                    ts.split_kb = (tp.k_blocks + splits - 1) / splits;
                    splits = (tp.k_blocks + ts.split_kb - 1) / ts.split_kb;
                    ts.split_row_stride = grid.y * kBM;
                    ts.out = g.splitk_scratch;
                    ts.out_pitch = g.n;
                    ts.alpha = 1.0f;
                    ts.beta = 0.0f;
                    ts.bias = nullptr;
                    grid.z = splits;
                    cudaError_t err = launch_tc<false, false, EPI_STORE_F32>(ma, mb, ts, grid, stream);
                    if (err != cudaSuccess)
                        return err;
                    const uint64_t quads = g.a_rows * (g.n / 4);
                    splitk_reduce_kernel<<<static_cast<unsigned>((quads + 255) / 256), 256, 0, stream>>>(
                        g.splitk_scratch, splits, static_cast<uint64_t>(ts.split_row_stride) * g.n, g.a_rows, g.n,
                        static_cast<float*>(g.out), g.out_pitch_elems, g.alpha == 0.0f ? 1.0f : g.alpha, g.beta, g.bias);
                    note_launch();
                    return cudaGetLastError();
                }
                return launch_tc<false, false, EPI_STORE_F32>(ma, mb, tp, grid, stream);
            }
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
