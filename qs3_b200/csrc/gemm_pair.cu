// NVFP4 grouped GEMMs on CTA pairs: tcgen05.mma.cta_group::2 instructions of 256 rows.
//
// The resident-A kernel of gemm.cu streams all of an expert's weights through every SM
// that holds one of its 128-row tiles, and the L2 -> SM path, not the tensor pipe, sets its
// pace. Here two CTAs of a cluster take a PAIR of row tiles of one expert (256 rows):
//
//   * each CTA keeps its own 128-row A panel (codes for the whole k <= 2048) in shared memory
//     and its scales in tensor memory, as before;
//   * per k block each CTA loads only HALF of the weight rows of a column tile -- the instruction
//     reads both halves, one from each CTA's shared memory -- so the weights cross L2 -> SM once
//     per 256 token rows instead of once per 128;
//   * the first CTA issues the instructions (kind::mxf4nvf4.block_scale, scale_vec::4X) for both;
//   * the weight-scale copies into tensor memory (tcgen05.cp) are issued by threads of their
//     own: issued by the MMA thread ahead of the MMAs that read them they stall the pipe for
//     ~50 cycles each (measured: 740 -> 939 cycles per k block with four copies), issued from
//     another thread they cost nothing. The threads hand scale buffers back and forth through
//     mbarriers (tcgen05.commit).
//
// Two shapes (PairShape):
//
//   gated (gate_up + SwiGLU + NVFP4 re-quantisation): column tiles of 256 accumulator columns (128
//     gate + 128 up features), 256 x 256 instructions, which reach a ~1.33x higher tensor-pipe ceiling
//     than 128-column ones (6.6 vs 5.0 PFLOP/s measured with the issue-loop probe). A 256-column f32
//     accumulator plus resident scales leaves no room in the 512 tensor-memory columns for a second
//     one, so the epilogue warps first DRAIN the accumulator into registers (128 values per thread),
//     hand it back to the MMA thread, and only then run SwiGLU + quantisation from registers while
//     the next column tile's MMAs run.
//   plain (down projection, bf16 out): column tiles of 128 columns and TWO accumulators. k is the
//     intermediate size there, a column tile is eight instructions long, and the hand-over of a single
//     accumulator would idle the pipe half of the time; the kernel is bound by its bf16 output, not by
//     the instruction rate. Tiles leave through two shared-memory staging buffers and TMA stores.
//
// No load uses cluster multicast: every CTA issues plain cp.async.bulk.tensor loads into its
// own shared memory (completion counted on the first CTA's barrier), so the kernel is fit
// for processes that run on several GPUs. Every tensor map covers this GPU's memory only.
//
// Work units: (pair tile, range of column tiles), walked by persistent clusters with a static
// stride. An expert with an odd number of row tiles ends in a "single": the second CTA then
// has no rows; it still provides its half of the weights.
//
//   warps 0-7  epilogue (two per tensor-memory lane quadrant, each half of the tile's columns)
//   warp 8     TMA producer (weight ring and A panels)
//   warp 9     MMA issuer (first CTA)     warps 10, 11  scale copiers (first CTA; 11 only for 256 columns)
//
//   TMEM  gated: [0,256) accumulator | plain: [0,128) and [128,256) accumulators
//         [256,384) A scales (k/64 x 4 columns) | [384,512) buffers of B scales, one per ring stage
//         (4 columns per 128 weight rows and 64 k elements)
//   smem  A panel k_blocks x 16 KB | A-scale staging k_blocks x 2 KB | ring of stages, each this CTA's
//         half of the weight codes of a 256-element k block + the scales of ALL the tile's weight rows
//         (gated 16 + 4 KB, plain 8 + 2 KB) | plain: two 32 KB bf16 staging buffers
//
// Every wait is bounded (tcgen05.cuh); on expiry the kernel records a code in the device
// error word and leaves through the normal teardown.
#include "tcgen05.cuh"

#include <cooperative_groups.h>

#include <algorithm>
#include <cstdlib>

namespace qs3 {

namespace {

using namespace tc;

constexpr int kPgThreads = 384;
constexpr uint32_t kPgMaxKBlocks = 8;
constexpr uint32_t kPgMaxStages = 8;
constexpr uint32_t kPgTmemCols = 512;

// Shape of a column tile. Gated (gate_up) problems use 256-column instructions and ONE accumulator;
// plain (down) problems use 128-column instructions and TWO accumulators: their k is short (the
// intermediate size), so a column tile is only a few instructions long and the hand-over of a
// single accumulator to the epilogue would idle the tensor pipe half of the time, while the
// lower issue rate of the narrower instruction does not matter for a kernel bound by its output.
template <bool GATED> struct PairShape {
    static constexpr uint32_t kBN = GATED ? 256u : 128u;             // accumulator columns per column tile
    static constexpr uint32_t kAccs = GATED ? 1u : 2u;               // accumulators in tensor memory
    // k blocks (256 elements) per ring stage. Every tcgen05 instruction and every barrier wait costs the one
    // issuing thread 50-100 cycles; with 128-column instructions (147 cycles of tensor pipe each) a stage of
    // four instructions plus its commits and waits takes that thread longer than the pipe needs, so plain
    // stages carry two k blocks (measured: down GEMM 0.150 -> 0.134 ms).
    static constexpr uint32_t kKbs = GATED ? 1u : 2u;
    // A panels in shared memory (and sets of A scales in tensor memory). Plain problems have a short k and
    // keep two: the next unit's panel is loaded while the current unit runs. The gated panel (k = 2048:
    // 128 KB) leaves room for one; it is refilled k block by k block behind the unit's last column tile.
    static constexpr uint32_t kPanels = GATED ? 1u : 2u;
    static constexpr uint32_t kKbCols = kBN / 8;                     // B-scale columns per k block (4 MMAs)
    static constexpr uint32_t kSlotCols = kKbs * kKbCols;            // ... per ring stage
    static constexpr uint32_t kSfbBufs = 128 / kSlotCols;            // ring stages the B-scale columns allow
    static constexpr uint32_t kCodeBytes = kBN / 2 * 128;            // this CTA's half of the weight rows, one k block
    static constexpr uint32_t kScaleBytes = kBN / 128 * kSfBytes;    // scales of all kBN weight rows, one k block
    static constexpr uint32_t kStageBytes = kKbs * (kCodeBytes + kScaleBytes); // codes of all k blocks, then scales
};

enum : uint32_t {
    ERR_PG_PANEL_FREE = 0x54000001u,
    ERR_PG_PANEL_FULL = 0x54000002u,
    ERR_PG_EMPTY = 0x54000003u,
    ERR_PG_FULL = 0x54000004u,
    ERR_PG_SF_READY = 0x54000006u,
    ERR_PG_SFA_READY = 0x54000007u,
    ERR_PG_ACC_EMPTY = 0x54000008u,
    ERR_PG_ACC_FULL = 0x54000009u,
};

// Measurement aid (QS3_PAIR_DBG bit 32): the first cluster's leader CTA stamps clock64() at the
// hand-over points of its first kTraceStages ring stages: [role][stage][event].
constexpr uint32_t kTraceStages = 192;
constexpr uint32_t kTraceEvents = 4;
constexpr uint32_t kTraceRoles = 4; // 0 producer, 1 scale copier, 2 MMA issuer, 3 epilogue warp 0 (per column tile)
__device__ unsigned long long g_pair_trace[kTraceRoles * kTraceStages * kTraceEvents];
// ... and every cluster's MMA thread the global timer (ns) when it starts and when it has issued its last
// unit, and how many units it took: [cluster][start, end, units]
constexpr uint32_t kTraceClusters = 128;
__device__ unsigned long long g_pair_spans[kTraceClusters * 3];

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void trace(bool on, uint32_t role, uint32_t stage, uint32_t event)
{
    if (on && stage < kTraceStages)
        g_pair_trace[(role * kTraceStages + stage) * kTraceEvents + event] = static_cast<unsigned long long>(clock64());
}

struct PairParams {
    TcParams tc;
    const int32_t* pair_expert;  // NULL: dense problem (pair tile p = rows [256 p, 256 p + 256))
    const int32_t* pair_row0;
    const int32_t* pair_nrows;
    const int32_t* pair_counts;  // [2]: full pairs (table filled from index 0 up), singles (from the top down)
    uint32_t pair_cap;           // entries of the pair tables
    uint32_t stages;
    uint32_t sfa_tiles_per_block; // 512-byte A-scale tiles per 128 rows (= k / 64)
    uint32_t sfb_tiles_per_group; // 512-byte B-scale tiles per expert
    uint32_t force_splits;        // measurement only (QS3_PAIR_SPLITS): work units per pair tile, 0 = automatic
    uint32_t dbg;                 // measurement only (QS3_PAIR_DBG): 1 no epilogue arithmetic / stores,
                                  // 2 no accumulator drain either, 4 no MMAs, 8 no weight-scale copies,
                                  // 16 L2 prefetch of the next column tile, 32 record the stage trace
                                  // (qs3_debug_pair_trace)
};

__device__ __forceinline__ uint32_t cluster_addr(const void* local, uint32_t cta_rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(cta_rank));
    return remote;
}

// TMA tile load of this CTA into its own shared memory; the bytes are counted on a barrier
// that may live in the other CTA of the pair. No multicast.
__device__ __forceinline__ void tma_load_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                              int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void tma_load_pair_3d(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

// The same boxes fetched into L2 only (no shared memory, no barrier): issued one column tile
// ahead so that the ring's loads find their data in L2 instead of waiting for HBM.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int c0, int c1)
{
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

// Arrival on a barrier of either CTA of the pair. CTA-scope release: what it publishes is that this
// warp's tensor-memory reads are complete (tcgen05.wait::ld + tcgen05.fence::before_thread_sync come
// first); a cluster-scope release would also wait for the warp's earlier global stores to be
// acknowledged, ~1000 cycles per column tile on the accumulator hand-back.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ void commit_pair(uint32_t bar_cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

// One commit that arrives on the barrier at the same shared-memory offset in BOTH CTAs of the pair
// (the multicast here is of the barrier arrival, not of a load): the issuing thread pays 50-100
// cycles per tcgen05 instruction, so one commit instead of two per ring stage matters.
__device__ __forceinline__ void commit_both(const void* local_bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
                     "r"(smem_u32(local_bar)),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
}

__device__ __forceinline__ void cp_scales_pair(uint32_t taddr, uint64_t sdesc)
{
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void mma_nvfp4_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc,
                                               uint32_t sfa, uint32_t sfb)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X"
                 " [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d),
                 "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb)
                 : "memory");
}

// 64 consecutive accumulator columns of this warp's 32 lanes -> 64 registers per thread
__device__ __forceinline__ void tc_ld64(uint32_t taddr, uint32_t* r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32"
        " {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
        " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31,"
        " %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47,"
        " %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
          "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
          "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
          "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}

// 64 accumulator values of one row -> 64 bf16 in row `r` of a 128-row x 128-byte staging sub-tile laid
// out with the 128-byte swizzle the TMA store expects (16-byte chunk c of row r sits at chunk c ^ (r & 7)).
__device__ __forceinline__ void stage_bf16_rows(const uint32_t (&v)[64], uint8_t* sub_tile, uint32_t r, float scale)
{
    uint8_t* row_smem = sub_tile + r * 128;
#pragma unroll
    for (uint32_t c = 0; c < 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            w[i] = pack_bf16x2(__uint_as_float(v[c * 8 + 2 * i]) * scale, __uint_as_float(v[c * 8 + 2 * i + 1]) * scale);
        *reinterpret_cast<uint4*>(row_smem + ((c ^ (r & 7u)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

struct Unit {
    int expert;
    int row0;   // first padded row of the pair tile
    int nrows;  // valid rows, 1..256
    uint32_t nt_begin, nt_end;
};

// Work units. A unit is a pair tile with a range of its column tiles; clusters take units u = cluster,
// cluster + clusters, ... Every thread derives the same schedule from the device-side tile counts:
//   * few pair tiles (less than four rounds of whole tiles): every tile is split into `splits` units
//     (2 or 4), so that all clusters have work;
//   * otherwise whole tiles, except the tiles of the last, partial round, which are split `tail_splits`
//     ways when that shortens the tail (22 left-over tiles on 74 clusters: one half-round of
//     half-tiles instead of one round of whole tiles). A split unit reloads its A panel.
struct Sched {
    uint32_t n_tiles;      // column tiles of a pair tile
    uint32_t whole;        // leading tiles taken whole (or every tile, `splits` ways)
    uint32_t splits;       // units per tile among the first `whole` tiles
    uint32_t tail_splits;  // units per tile after them
    uint32_t total_units;
};

__device__ __forceinline__ Sched make_sched(uint32_t pair_tiles, uint32_t n_tiles, uint32_t clusters, uint32_t force)
{
    Sched sc;
    sc.n_tiles = n_tiles;
    sc.splits = 1;
    sc.tail_splits = 1;
    sc.whole = pair_tiles;
    if (force != 0) {
        sc.splits = force;
    } else if (pair_tiles < 4 * clusters) {
        while (sc.splits * 2 <= n_tiles && n_tiles % (sc.splits * 2) == 0 && pair_tiles * sc.splits < 4 * clusters)
            sc.splits *= 2;
    } else {
        const uint32_t rest = pair_tiles % clusters;
        sc.whole = pair_tiles - rest;
        // cost of the tail in sixteenths of a whole-tile round, plus one sixteenth per reload of the panel
        uint32_t best = 0xffffffffu;
        for (uint32_t ts = 1; ts <= 4 && ts <= n_tiles && rest != 0; ts *= 2) {
            if (n_tiles % ts != 0)
                continue;
            const uint32_t cost = (rest * ts + clusters - 1) / clusters * (16 / ts) + (ts - 1);
            if (cost < best) {
                best = cost;
                sc.tail_splits = ts;
            }
        }
    }
    sc.total_units = sc.whole * sc.splits + (pair_tiles - sc.whole) * sc.tail_splits;
    return sc;
}

__device__ __forceinline__ bool load_unit(const PairParams& p, uint32_t u, const Sched& sc, Unit* out)
{
    if (u >= sc.total_units)
        return false;
    uint32_t tile, split, parts;
    if (u < sc.whole * sc.splits) {
        parts = sc.splits;
        tile = u / parts;
        split = u % parts;
    } else {
        parts = sc.tail_splits;
        const uint32_t v = u - sc.whole * sc.splits;
        tile = sc.whole + v / parts;
        split = v % parts;
    }
    const uint32_t nt_per_unit = sc.n_tiles / parts;
    if (p.pair_expert != nullptr) {
        const uint32_t full = static_cast<uint32_t>(p.pair_counts[0]);
        const uint32_t idx = tile < full ? tile : p.pair_cap - 1 - (tile - full);
        out->expert = p.pair_expert[idx];
        out->row0 = p.pair_row0[idx];
        out->nrows = p.pair_nrows[idx];
    } else {
        out->expert = 0;
        out->row0 = static_cast<int>(tile) * 256;
        out->nrows = min(256, static_cast<int>(p.tc.dense_rows) - out->row0);
    }
    out->nt_begin = split * nt_per_unit;
    out->nt_end = out->nt_begin + nt_per_unit;
    return true;
}

// TMA coordinates of what one CTA streams for a column tile (see the producer).
struct Coords {
    int b1, b2; // weight rows: gated (row within the gate / up half, 2 * expert), plain (row, unused)
    int sf2;    // first of the tile's two 128-row blocks in the scale-tile map
};

template <bool GATED>
__device__ __forceinline__ Coords tile_coords(const TcParams& p, const PairParams& pp, int expert, uint32_t nt,
                                              uint32_t rank)
{
    using Shape = PairShape<GATED>;
    const uint32_t it = 2 * nt + rank;
    Coords c;
    if (GATED) {
        c.b1 = static_cast<int>(it * 64);
        c.b2 = 2 * expert;
    } else {
        c.b1 = expert * static_cast<int>(p.b_rows) + static_cast<int>(it * (Shape::kBN / 2));
        c.b2 = 0;
    }
    c.sf2 = static_cast<int>(expert * (p.b_rows / 128) + (Shape::kBN / 128) * nt);
    return c;
}

template <bool GATED, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPgThreads, 1)
gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                       const __grid_constant__ CUtensorMap map_o, const PairParams pp)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = cluster.block_rank();
    const TcParams& p = pp.tc;
    const uint32_t kb_count = p.k_blocks;
    using Shape = PairShape<GATED>;
    constexpr uint32_t kPgBN = Shape::kBN;
    constexpr uint32_t kAccs = Shape::kAccs;
    constexpr uint32_t kPgStageBytes = Shape::kStageBytes;
    constexpr uint32_t kKbs = Shape::kKbs;
    const uint32_t stages = pp.stages; // ring stages = weight-scale buffers in tensor memory (<= Shape::kSfbBufs)

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr uint32_t nb = Shape::kPanels; // A panels in shared memory (unit i uses panel i % nb)
    uint8_t* a_panel = smem;                                  // [nb][kb_count] 16 KB tiles
    uint8_t* sfa_stage = a_panel + nb * kb_count * kTileBytes; // [nb][kb_count] 2 KB
    uint8_t* ring = sfa_stage + nb * kb_count * kSfBytes;
    // bf16 output tiles leave through shared memory and TMA stores: four 128-row x 128-byte sub-tiles
    uint8_t* staging = ring + stages * kPgStageBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + (GATED ? 0 : 4 * kTileBytes));
    uint64_t* empty_bar = full_bar + kPgMaxStages;
    uint64_t* sf_ready = empty_bar + kPgMaxStages;
    // per panel and k block, index panel * kb_count + kb (nb * kb_count <= kPgMaxKBlocks):
    uint64_t* panel_full = sf_ready + kPgMaxStages;        // A codes + A scales of both CTAs landed
    uint64_t* panel_free = panel_full + kPgMaxKBlocks;     // the unit's last MMAs on it are done
    uint64_t* sfa_ready = panel_free + kPgMaxKBlocks;      // A scales are in tensor memory
    uint64_t* acc_full = sfa_ready + kPgMaxKBlocks;        // [kAccs]
    uint64_t* acc_empty = acc_full + 2;                    // [kAccs]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* go_flag = tmem_slot + 2; // plain tiles: the epilogue warps' common "carry on" decision

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
            mbar_init(&sf_ready[s], kPgBN / 128); // one scale copier per 128 weight rows
        }
        for (uint32_t kb = 0; kb < nb * kb_count; ++kb) {
            mbar_init(&panel_full[kb], 1);
            mbar_init(&panel_free[kb], 1);
            mbar_init(&sfa_ready[kb], 1);
        }
        for (uint32_t b = 0; b < kAccs; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 16); // eight epilogue warps in each CTA
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    cluster.sync(); // both CTAs resident and their barriers initialised before anything is signalled
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kPgTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster.sync();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sfa = tmem_base + 256;
    const uint32_t tmem_sfb = tmem_base + 384;

    constexpr uint32_t kFeat = GATED ? kPgBN / 2 : kPgBN; // output features per column tile
    const uint32_t n_tiles = (p.n + kFeat - 1) / kFeat;
    const uint32_t pair_tiles = pp.pair_expert != nullptr
        ? static_cast<uint32_t>(pp.pair_counts[0] + pp.pair_counts[1])
        : (p.dense_rows + 255) / 256;
    const uint32_t cluster_id = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    const bool tr = (pp.dbg & 32u) != 0 && blockIdx.x == 0;
    const Sched sc = make_sched(pair_tiles, n_tiles, clusters, pp.force_splits);
    const uint32_t total_units = sc.total_units;

    if (warp == 8) {
        // ------------------------------------------------------------ producer --
        // One thread feeds two streams. The weight ring runs ahead across unit boundaries (it does not
        // depend on the panel). The A panels go k block by k block: block kb of the next unit's panel is
        // loaded as soon as the last column tile of the current unit is done with block kb, so a panel
        // trails the previous unit's last column tile by one k block instead of waiting for its end. The
        // panel stream is polled, never waited for, so that it cannot hold up the ring.
        if (lane == 0) {
            uint32_t p_unit = cluster_id, p_no = 0, p_kb = 0, p_slot0 = 0, p_par = 0;
            Unit pu;
            bool p_have = load_unit(pp, p_unit, sc, &pu);
            const auto pump_panel = [&]() {
                // panel p_no goes into buffer p_no % nb (first slot p_slot0), whose previous user was panel
                // p_no - nb; p_par is the parity of (p_no / nb)
                while (p_have && mbar_test_wait(&panel_free[p_slot0 + p_kb], p_par ^ 1)) {
                    const int my_row0 = pu.row0 + static_cast<int>(rank * 128);
                    const uint32_t slot = p_slot0 + p_kb;
                    if (rank == 0)
                        mbar_expect_tx(&panel_full[slot], (pu.nrows > 128 ? 2u : 1u) * (kTileBytes + kSfBytes));
                    if (pu.nrows > static_cast<int>(rank * 128)) {
                        const uint32_t pbar = cluster_addr(&panel_full[slot], 0);
                        tma_load_pair(a_panel + slot * kTileBytes, &map_a, pbar, static_cast<int>(p_kb) * 128, my_row0);
                        tma_load_pair(sfa_stage + slot * kSfBytes, &map_sfa, pbar, 0,
                                      static_cast<int>((my_row0 >> 7) * pp.sfa_tiles_per_block + 4 * p_kb));
                    }
                    if (++p_kb == kb_count) {
                        p_kb = 0;
                        ++p_no;
                        p_slot0 += kb_count;
                        if (p_slot0 == nb * kb_count) {
                            p_slot0 = 0;
                            p_par ^= 1;
                        }
                        p_unit += clusters;
                        p_have = load_unit(pp, p_unit, sc, &pu);
                    }
                }
            };
            // bounded wait for a ring slot that keeps the panel stream going
            const auto wait_slot = [&](uint64_t* bar, uint32_t parity) -> bool {
                if (mbar_test_wait(bar, parity))
                    return true;
                const uint64_t start = clock64();
                uint32_t spins = 0;
                while (!mbar_test_wait(bar, parity)) {
                    pump_panel();
                    if ((++spins & 15u) != 0)
                        continue;
                    if (*abort_flag != 0)
                        return false;
                    if (static_cast<uint64_t>(clock64()) - start > kWaitCycles) {
                        *abort_flag = 1;
                        atomicCAS(p.err, 0u, static_cast<uint32_t>(ERR_PG_EMPTY));
                        return false;
                    }
                }
                return true;
            };
            uint32_t s = 0, ph = 0, tsi = 0;
            bool ok = true;
            Unit un, next;
            pump_panel();
            for (uint32_t u = cluster_id; ok && load_unit(pp, u, sc, &un); u += clusters) {
                const bool have_next = load_unit(pp, u + clusters, sc, &next);
                for (uint32_t nt = un.nt_begin; ok && nt < un.nt_end; ++nt) {
                    // What this CTA streams for column tile nt: 128 of the tile's 256 weight rows
                    // ("interleaved tile" 2 nt + rank: for gated problems 64 gate rows and their 64 up rows, one
                    // 3-D box) and the scales of all 256 rows (two row blocks of four 512-byte tiles, one 3-D box).
                    const Coords cur = tile_coords<GATED>(p, pp, un.expert, nt, rank);
                    // one column tile ahead (the next unit's first one after this unit's last), into L2
                    Coords ahead = cur;
                    bool pf = (pp.dbg & 16u) != 0;
                    if (nt + 1 < un.nt_end)
                        ahead = tile_coords<GATED>(p, pp, un.expert, nt + 1, rank);
                    else if (have_next)
                        ahead = tile_coords<GATED>(p, pp, next.expert, next.nt_begin, rank);
                    else
                        pf = false;
                    for (uint32_t kb0 = 0; kb0 < kb_count; kb0 += kKbs) {
                        if (!wait_slot(&empty_bar[s], ph ^ 1)) {
                            ok = false;
                            break;
                        }
                        trace(tr, 0, tsi, 0);
                        uint8_t* sb = ring + s * kPgStageBytes;
                        if (rank == 0)
                            mbar_expect_tx(&full_bar[s], 2 * kPgStageBytes);
                        const uint32_t fbar = cluster_addr(&full_bar[s], 0);
#pragma unroll
                        for (uint32_t q = 0; q < kKbs; ++q) {
                            const uint32_t kb = kb0 + q;
                            const int c0 = static_cast<int>(kb) * 128;
                            if (GATED)
                                tma_load_pair_3d(sb + q * Shape::kCodeBytes, &map_b, fbar, c0, cur.b1, cur.b2);
                            else
                                tma_load_pair(sb + q * Shape::kCodeBytes, &map_b, fbar, c0, cur.b1);
                            tma_load_pair_3d(sb + kKbs * Shape::kCodeBytes + q * Shape::kScaleBytes, &map_sfb, fbar, 0,
                                             static_cast<int>(4 * kb), cur.sf2);
                            if (pf) {
                                if (GATED)
                                    tma_prefetch_3d(&map_b, c0, ahead.b1, ahead.b2);
                                else
                                    tma_prefetch_2d(&map_b, c0, ahead.b1);
                                tma_prefetch_3d(&map_sfb, 0, static_cast<int>(4 * kb), ahead.sf2);
                            }
                        }
                        trace(tr, 0, tsi++, 1);
                        pump_panel();
                        if (++s == stages) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                }
            }
            // The ring can be issued to its end while the MMAs are still a few units behind (short
            // units: fewer stages per unit than the ring holds); the panels of those last units are still
            // to come, so keep feeding the panel stream until its last block is out.
            uint64_t start = clock64();
            uint32_t seen_no = p_no, seen_kb = p_kb;
            while (ok && p_have) {
                pump_panel();
                if (p_no != seen_no || p_kb != seen_kb) { // progress: restart the clock
                    seen_no = p_no;
                    seen_kb = p_kb;
                    start = clock64();
                } else if (*abort_flag != 0) {
                    break;
                } else if (static_cast<uint64_t>(clock64()) - start > kWaitCycles) {
                    *abort_flag = 1;
                    atomicCAS(p.err, 0u, static_cast<uint32_t>(ERR_PG_PANEL_FREE));
                    break;
                }
            }
        }
    } else if (warp == 11) {
        // ------------------------------------------- second scale copier --
        // tcgen05.cp costs its issuing thread 50-70 cycles apiece; the eight copies of a stage's B scales
        // (plus four of A scales in a unit's first column tile) from one thread take longer than the
        // stage's four MMAs, so the two 128-row halves of the B scales have a copier thread each.
        if (kPgBN == 256 && rank == 0 && lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            Unit un;
            for (uint32_t u = cluster_id; ok && load_unit(pp, u, sc, &un); u += clusters) {
                for (uint32_t nt = un.nt_begin; ok && nt < un.nt_end; ++nt) {
                    for (uint32_t kb0 = 0; kb0 < kb_count; kb0 += kKbs) {
                        if (!mbar_wait<true>(&full_bar[s], ph, abort_flag, p.err, ERR_PG_FULL)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        // the second 128 weight rows of every k block of the stage
                        const uint32_t sf_smem = smem_u32(ring + s * kPgStageBytes) + kKbs * Shape::kCodeBytes + kSfBytes;
                        if (!(pp.dbg & 8u)) {
#pragma unroll
                            for (uint32_t q = 0; q < kKbs; ++q)
#pragma unroll
                                for (uint32_t j = 0; j < 4; ++j)
                                    cp_scales_pair(tmem_sfb + Shape::kSlotCols * s + Shape::kKbCols * q + 8 * j + 4,
                                                   scale_desc(sf_smem + q * Shape::kScaleBytes + j * 512));
                        }
                        commit_pair(cluster_addr(&sf_ready[s], 0));
                        if (++s == stages) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                }
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------- MMA issuer --
        if (rank == 0 && lane == 0) {
            constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((kPgBN >> 3) << 17) | ((256u >> 4) << 24);
            const uint32_t a_addr = smem_u32(a_panel);
            uint32_t s = 0, ph = 0, unit_no = 0, tile_no = 0, sfi = 0;
            bool ok = true;
            Unit un;
            const bool spans = (pp.dbg & 32u) != 0 && cluster_id < kTraceClusters;
            if (spans)
                g_pair_spans[cluster_id * 3] = global_ns();
            for (uint32_t u = cluster_id; ok && load_unit(pp, u, sc, &un); u += clusters, ++unit_no) {
                const bool more = u + nb * clusters < total_units; // a later unit of this cluster reuses the panel
                const uint32_t pslot = (unit_no % nb) * kb_count;   // first barrier / tile / scale slot of the panel
                for (uint32_t nt = un.nt_begin; ok && nt < un.nt_end; ++nt, ++tile_no) {
                    const uint32_t buf = tile_no % kAccs, use = tile_no / kAccs;
                    if (!mbar_wait<true>(&acc_empty[buf], (use & 1) ^ 1, abort_flag, p.err, ERR_PG_ACC_EMPTY)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t tmem_acc = tmem_base + buf * kPgBN;
                    const bool first = nt == un.nt_begin, last = nt + 1 == un.nt_end;
                    for (uint32_t kb0 = 0; kb0 < kb_count; kb0 += kKbs, ++sfi) {
                        trace(tr, 2, sfi, 0);
                        // A scales of the stage's k blocks (first column tile of a unit; implies the A codes landed)
                        if (first) {
                            for (uint32_t q = 0; ok && q < kKbs; ++q)
                                ok = mbar_wait<true>(&sfa_ready[pslot + kb0 + q], (unit_no / nb) & 1, abort_flag, p.err,
                                                     ERR_PG_SFA_READY);
                            if (!ok)
                                break;
                        }
                        trace(tr, 2, sfi, 1);
                        // both copiers are done with the stage's B scales (they waited for the stage's loads)
                        if (!mbar_wait<true>(&sf_ready[s], ph, abort_flag, p.err, ERR_PG_SF_READY)) {
                            ok = false;
                            break;
                        }
                        trace(tr, 2, sfi, 2);
                        tc_fence_after();
                        if (!(pp.dbg & 4u)) {
#pragma unroll
                            for (uint32_t q = 0; q < kKbs; ++q) {
                                const uint32_t kb = kb0 + q;
                                const uint64_t da = operand_desc(a_addr + (pslot + kb) * kTileBytes);
                                const uint64_t db = operand_desc(smem_u32(ring + s * kPgStageBytes) + q * Shape::kCodeBytes);
#pragma unroll
                                for (uint32_t j = 0; j < 4; ++j)
                                    mma_nvfp4_pair(tmem_acc, da + 2 * j, db + 2 * j, kIdesc, (kb > 0 || j > 0) ? 1u : 0u,
                                                   tmem_sfa + 16 * (pslot + kb) + 4 * j,
                                                   tmem_sfb + Shape::kSlotCols * s + Shape::kKbCols * q + (kPgBN / 32) * j);
                            }
                        }
                        // the stage's shared memory and its scale buffer in tensor memory are free again
                        commit_both(&empty_bar[s]);
                        if (last && more) {
#pragma unroll
                            for (uint32_t q = 0; q < kKbs; ++q)
                                commit_both(&panel_free[pslot + kb0 + q]);
                        }
                        trace(tr, 2, sfi, 3);
                        if (++s == stages) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                    if (ok)
                        commit_both(&acc_full[buf]);
                }
            }
            if (spans) {
                g_pair_spans[cluster_id * 3 + 1] = global_ns();
                g_pair_spans[cluster_id * 3 + 2] = unit_no;
            }
        }
    } else if (warp == 10) {
        // -------------------------------------------------------- scale copier --
        // Same order as the MMA issuer consumes: per stage, in a unit's first column tile the A scales of
        // the stage's k block first (both CTAs' staging -> their own tensor memory), then the stage's B scales.
        if (rank == 0 && lane == 0) {
            uint32_t s = 0, ph = 0, unit_no = 0, sfi = 0;
            bool ok = true;
            Unit un;
            for (uint32_t u = cluster_id; ok && load_unit(pp, u, sc, &un); u += clusters, ++unit_no) {
                for (uint32_t nt = un.nt_begin; ok && nt < un.nt_end; ++nt) {
                    for (uint32_t kb0 = 0; kb0 < kb_count; kb0 += kKbs, ++sfi) {
                        trace(tr, 1, sfi, 0);
                        if (nt == un.nt_begin) {
                            for (uint32_t q = 0; ok && q < kKbs; ++q) {
                                const uint32_t slot = (unit_no % nb) * kb_count + kb0 + q;
                                if (!mbar_wait<true>(&panel_full[slot], (unit_no / nb) & 1, abort_flag, p.err,
                                                     ERR_PG_PANEL_FULL)) {
                                    ok = false;
                                    break;
                                }
                                tc_fence_after();
#pragma unroll
                                for (uint32_t j = 0; j < 4; ++j)
                                    cp_scales_pair(tmem_sfa + 16 * slot + 4 * j,
                                                   scale_desc(smem_u32(sfa_stage) + slot * kSfBytes + j * 512));
                                commit_pair(cluster_addr(&sfa_ready[slot], 0));
                            }
                            if (!ok)
                                break;
                        }
                        if (!mbar_wait<true>(&full_bar[s], ph, abort_flag, p.err, ERR_PG_FULL)) {
                            ok = false;
                            break;
                        }
                        trace(tr, 1, sfi, 1);
                        // (the stage was refilled, so the MMAs that read its scale buffer in tensor memory last
                        // time round are done: the buffer may be overwritten)
                        trace(tr, 1, sfi, 2);
                        tc_fence_after();
                        const uint32_t sf_smem = smem_u32(ring + s * kPgStageBytes) + kKbs * Shape::kCodeBytes;
                        if (!(pp.dbg & 8u)) {
#pragma unroll
                            for (uint32_t q = 0; q < kKbs; ++q)
#pragma unroll
                                for (uint32_t j = 0; j < 4; ++j)
                                    cp_scales_pair(tmem_sfb + Shape::kSlotCols * s + Shape::kKbCols * q + (kPgBN / 32) * j,
                                                   scale_desc(sf_smem + q * Shape::kScaleBytes + j * 512));
                        }
                        commit_pair(cluster_addr(&sf_ready[s], 0));
                        trace(tr, 1, sfi, 3);
                        if (++s == stages) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue --
        // warp w reads lane quadrant w % 4 and columns [128 (w / 4), +128) = "interleaved tile"
        // 2 nt + w / 4: 64 gate columns then their 64 up columns
        const uint32_t quad = warp & 3, half = warp >> 2;
        const uint32_t lane_base = (quad * 32) << 16;
        const uint32_t acc_empty_leader0 = cluster_addr(&acc_empty[0], 0);
        const uint32_t acc_empty_leader1 = cluster_addr(&acc_empty[kAccs - 1], 0);
        uint32_t tile_no = 0;
        Unit un;
        bool ok = true;
        for (uint32_t u = cluster_id; ok && load_unit(pp, u, sc, &un); u += clusters) {
            const int my_row0 = un.row0 + static_cast<int>(rank * 128);
            const int my_nrows = min(128, un.nrows - static_cast<int>(rank * 128));
            const int r = static_cast<int>(quad * 32 + lane);
            const bool row_ok = r < my_nrows;
            const uint64_t grow = static_cast<uint64_t>(my_row0) + r;
            float scale = p.alpha == 0.0f ? 1.0f : p.alpha;
            float scale_up = scale;
            if (p.group_scale != nullptr)
                scale *= p.group_scale[un.expert];
            scale_up *= p.group_scale_up != nullptr ? p.group_scale_up[un.expert]
                                                    : (p.group_scale != nullptr ? p.group_scale[un.expert] : 1.0f);
            for (uint32_t nt = un.nt_begin; nt < un.nt_end; ++nt, ++tile_no) {
                trace(tr && threadIdx.x == 0, 3, tile_no, 0);
                const uint32_t buf = tile_no % kAccs, use = tile_no / kAccs;
                const bool ready = __all_sync(
                    0xffffffffu, mbar_wait(&acc_full[buf], use & 1, abort_flag, p.err, ERR_PG_ACC_FULL));
                // Gated tiles use no block-wide barrier below, so a warp whose wait gave up may leave at once.
                // Plain tiles synchronise the eight epilogue warps twice per tile: there the decision to
                // stop is taken by one thread and read by all AFTER the first barrier, so that no warp can
                // be left waiting at a barrier the others have walked away from.
                if (GATED && !ready) {
                    ok = false;
                    break;
                }
                trace(tr && threadIdx.x == 0, 3, tile_no, 1);
                tc_fence_after();
                // gated: this warp's 128 columns (64 gate, 64 up); plain: its 64 of the tile's 128 columns
                uint32_t va[64], vb[GATED ? 64 : 1];
                const uint32_t acc_addr = tmem_base + buf * kPgBN + lane_base;
                if (ready && !(pp.dbg & 2u)) {
                    if constexpr (GATED) {
                        tc_ld64(acc_addr + half * 128, va);
                        tc_ld64(acc_addr + half * 128 + 64, vb);
                    } else {
                        tc_ld64(acc_addr + half * 64, va);
                    }
                    tc_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i)
                        va[i] = 0;
#pragma unroll
                    for (int i = 0; i < (GATED ? 64 : 1); ++i)
                        vb[i] = 0;
                }
                // the accumulator is in registers: hand it back before the arithmetic
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive_cluster(buf == 0 ? acc_empty_leader0 : acc_empty_leader1);
                trace(tr && threadIdx.x == 0, 3, tile_no, 2);
                const uint32_t it = 2 * nt + half; // 64 output features [64 it, 64 it + 64)
                if (pp.dbg & 1u)
                    continue;
                if constexpr (GATED && EPI == EPI_SWIGLU_NVFP4) {
                    if (!row_ok || it * 64 >= p.n)
                        continue;
                    uint32_t sf_word = 0;
                    uint8_t* o = static_cast<uint8_t*>(p.out) + grow * p.out_pitch + it * 32;
#pragma unroll
                    for (uint32_t c = 0; c < 4; ++c) {
                        float act[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float g = __uint_as_float(va[c * 16 + i]) * scale;
                            const float up = __uint_as_float(vb[c * 16 + i]) * scale_up;
                            act[i] = __fdividef(g, 1.0f + __expf(-g)) * up;
                        }
                        uint32_t lo, hi;
                        const uint8_t code = quantize_block16(act, p.out_global, &lo, &hi);
                        sf_word |= static_cast<uint32_t>(code) << (8 * c);
                        *reinterpret_cast<uint2*>(o + c * 8) = make_uint2(lo, hi);
                    }
                    // 64 features = one k group of the next GEMM: its four scale bytes are one word
                    *reinterpret_cast<uint32_t*>(p.out_sf + tiled_scale_offset(grow, 4ull * it, p.out_kgroups))
                        = sf_word;
                } else {
                    // plain tile: bf16, staged in shared memory (128-byte swizzle) and written with TMA stores.
                    // This warp holds columns [64 half, +64) of rows [32 quad, +32): sub-tile `half` of the
                    // staging buffer that belongs to this accumulator. Every row of the CTA's tile is written:
                    // rows past the segment's end are padding rows of the same expert, rows past the tensor are
                    // clipped by the TMA unit. A CTA without rows (the second CTA of a single) stores nothing.
                    const bool store = my_nrows > 0;
                    const bool issuer = warp == 0 && lane == 0;
                    uint8_t* stage_buf = staging + buf * 2 * kTileBytes;
                    if (issuer) { // the stores of the tile before last have finished reading this staging buffer
                        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        *go_flag = (ready && *abort_flag == 0) ? 1u : 0u;
                    }
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                    if (*go_flag == 0) {
                        ok = false;
                        break;
                    }
                    if (store)
                        stage_bf16_rows(va, stage_buf + half * kTileBytes, static_cast<uint32_t>(r), scale);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                    if (issuer && store) {
                        const int n0 = static_cast<int>(nt * kPgBN);
#pragma unroll
                        for (int sub = 0; sub < 2; ++sub)
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                             reinterpret_cast<uint64_t>(&map_o)),
                                         "r"(smem_u32(stage_buf + sub * kTileBytes)), "r"(n0 + sub * 64), "r"(my_row0)
                                         : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            }
        }
    }

    if (!GATED && threadIdx.x == 0)
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); // stores done before shared memory goes away
    tc_fence_before();
    cluster.sync(); // the pair's tensor memory is idle in both CTAs
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPgTmemCols)
                     : "memory");
    }
}


} // namespace

// Map over a buffer of 512-byte scale tiles: [tiles, 128 x u32], box = `box_tiles` whole tiles.
bool make_scale_tile_map(CUtensorMap* map, const void* base, uint64_t tiles, uint32_t box_tiles);
// 3-D maps: scale tiles as [row blocks, k groups, 128 x u32] with a box of two row blocks x four k groups;
// gated weights [groups * 2 halves, inter rows, k bytes] with a box of 64 gate rows + their 64 up rows.
bool make_scale_block_map(CUtensorMap* map, const void* base, uint64_t row_blocks, uint32_t kgroups,
                          uint32_t box_blocks = 2);
bool make_gated_weight_map(CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t inter,
                           uint64_t groups, uint64_t pitch_bytes, uint32_t box_halves = 2);

namespace {

template <bool GATED, int EPI>
cudaError_t launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& msa, const CUtensorMap& msb,
                        const CUtensorMap& mo, PairParams pp, uint32_t max_units, cudaStream_t stream)
{
    constexpr size_t kSmemBudget = 227 * 1024 - 1024 /* alignment slack */ - 1024 /* barriers */;
    constexpr uint32_t kPgStageBytes = PairShape<GATED>::kStageBytes;
    const size_t one_panel = static_cast<size_t>(pp.tc.k_blocks) * (kTileBytes + kSfBytes);
    const size_t staging = GATED ? 0 : 4 * kTileBytes;
    const size_t panel = PairShape<GATED>::kPanels * one_panel + staging;
    if (PairShape<GATED>::kPanels * pp.tc.k_blocks > kPgMaxKBlocks || panel + 2 * kPgStageBytes > kSmemBudget)
        return cudaErrorInvalidConfiguration;
    uint32_t stages = static_cast<uint32_t>((kSmemBudget - panel) / kPgStageBytes);
    stages = std::min<uint32_t>(stages, PairShape<GATED>::kSfbBufs);
    if (const char* v = std::getenv("QS3_PAIR_STAGES"))
        stages = std::max(2u, std::min<uint32_t>(stages, static_cast<uint32_t>(std::atoi(v))));
    if (stages < 2)
        return cudaErrorInvalidConfiguration;
    pp.stages = stages;
    const size_t smem = panel + static_cast<size_t>(stages) * kPgStageBytes + 1024 + 1024;
    auto kernel = gemm_nvfp4_pair_kernel<GATED, EPI>;
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
    const uint32_t clusters = std::max(1u, std::min(max_units, device_sm_count() / 2));
    kernel<<<2 * clusters, kPgThreads, smem, stream>>>(ma, mb, msa, msb, mo, pp);
    note_launch();
    return cudaGetLastError();
}

} // namespace

bool nvfp4_pair_gemm_supported(const GemmProblem& g)
{
    if (!g.nvfp4 || g.k % 256 != 0 || g.k / 256 > kPgMaxKBlocks)
        return false;
    if (g.tile_expert != nullptr && (g.pair_expert == nullptr || g.tile_rows != 128))
        return false;
    const bool aligned = (reinterpret_cast<uintptr_t>(g.a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(g.b) & 15u) == 0
        && g.a_pitch_bytes % 16 == 0 && g.b_pitch_bytes % 16 == 0
        && (reinterpret_cast<uintptr_t>(g.a_scale_tiled) & 15u) == 0
        && (reinterpret_cast<uintptr_t>(g.b_scale_tiled) & 15u) == 0;
    if (!aligned)
        return false;
    if (g.gated)
        return g.epilogue == EPI_SWIGLU_NVFP4 && g.n % 128 == 0;
    return g.epilogue == EPI_STORE_BF16 && g.beta == 0.0f && g.n % 128 == 0
        && (g.k / 256) % PairShape<false>::kKbs == 0 && g.k <= 768 /* two panels + staging + a ring of two stages */
        && (reinterpret_cast<uintptr_t>(g.out) & 15u) == 0 && (g.out_pitch_elems * 2) % 16 == 0;
}

cudaError_t launch_nvfp4_pair_gemm(const GemmProblem& g, cudaStream_t stream, const char** why)
{
    PairParams pp {};
    TcParams& tp = pp.tc;
    tp.n = g.n;
    tp.b_rows = g.gated ? 2 * g.n : g.n;
    tp.kgroups = g.k / 64;
    tp.k_blocks = g.k / 256;
    tp.dense_rows = static_cast<uint32_t>(g.a_rows);
    tp.out = g.out;
    tp.out_pitch = g.out_pitch_elems;
    tp.out_sf = g.out_scale_tiled;
    tp.out_kgroups = g.n / 64;
    tp.alpha = g.alpha;
    tp.group_scale = g.group_scale;
    tp.group_scale_up = g.group_scale_up;
    tp.out_global = g.out_global_scale == 0.0f ? 1.0f : g.out_global_scale;
    tp.err = device_error_word();
    pp.pair_expert = g.tile_expert != nullptr ? g.pair_expert : nullptr;
    pp.pair_row0 = g.pair_row0;
    pp.pair_nrows = g.pair_nrows;
    pp.pair_counts = g.pair_counts;
    pp.pair_cap = g.max_tiles;
    pp.sfa_tiles_per_block = tp.kgroups;
    pp.sfb_tiles_per_group = (tp.b_rows / 128) * tp.kgroups;
    static const uint32_t dbg = [] {
        const char* v = std::getenv("QS3_PAIR_DBG");
        return v != nullptr ? static_cast<uint32_t>(std::atoi(v)) : 0u;
    }();
    pp.dbg = dbg;
    const uint32_t n_tiles = tp.b_rows / (g.gated ? PairShape<true>::kBN : PairShape<false>::kBN);
    static const uint32_t force_splits = [] {
        const char* v = std::getenv("QS3_PAIR_SPLITS");
        return v != nullptr ? static_cast<uint32_t>(std::atoi(v)) : 0u;
    }();
    pp.force_splits = (force_splits == 1 || force_splits == 2 || force_splits == 4) && n_tiles % force_splits == 0
        ? force_splits : 0;

    CUtensorMap ma, mb, msa, msb;
    const uint64_t b_total_rows = static_cast<uint64_t>(g.groups) * tp.b_rows;
    const uint64_t sfa_tiles = ((g.a_rows + 127) / 128) * tp.kgroups;
    const uint64_t sfb_tiles = static_cast<uint64_t>(g.groups) * pp.sfb_tiles_per_group;
    if (!make_operand_map(&ma, true, g.a, g.k / 2, g.a_rows, g.a_pitch_bytes, 128)
        || !(g.gated ? make_gated_weight_map(&mb, g.b, g.k / 2, g.n, g.groups, g.b_pitch_bytes)
                     : make_operand_map(&mb, true, g.b, g.k / 2, b_total_rows, g.b_pitch_bytes,
                                        PairShape<false>::kBN / 2))
        || !make_scale_tile_map(&msa, g.a_scale_tiled, sfa_tiles, 4)
        || !make_scale_block_map(&msb, g.b_scale_tiled, sfb_tiles / tp.kgroups, tp.kgroups,
                                 g.gated ? PairShape<true>::kBN / 128 : PairShape<false>::kBN / 128)) {
        if (why != nullptr)
            *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    // upper bound of the work units (the kernel splits a pair tile's column tiles at most n_tiles ways)
    const uint32_t max_units = (g.tile_expert != nullptr ? g.max_tiles : static_cast<uint32_t>((g.a_rows + 255) / 256))
        * n_tiles;
    if (g.gated)
        return launch_pair<true, EPI_SWIGLU_NVFP4>(ma, mb, msa, msb, ma, pp, max_units, stream);
    CUtensorMap mo;
    if (!make_operand_map(&mo, false, g.out, g.n, g.a_rows, g.out_pitch_elems * 2, 128)) {
        if (why != nullptr)
            *why = "cuTensorMapEncodeTiled failed";
        return cudaErrorInvalidValue;
    }
    return launch_pair<false, EPI_STORE_BF16>(ma, mb, msa, msb, mo, pp, max_units, stream);
}

} // namespace qs3

extern "C" qsfi_status qs3_debug_pair_trace(uint64_t* out, uint32_t capacity, uint32_t* count)
{
    using namespace qs3;
    constexpr uint32_t total = kTraceRoles * kTraceStages * kTraceEvents;
    if (out == nullptr || count == nullptr || capacity < total)
        return QSFI_STATUS_INVALID_ARGUMENT;
    if (cudaDeviceSynchronize() != cudaSuccess
        || cudaMemcpyFromSymbol(out, g_pair_trace, total * sizeof(uint64_t)) != cudaSuccess)
        return QSFI_STATUS_CUDA_ERROR;
    *count = total;
    return QSFI_STATUS_OK;
}

extern "C" qsfi_status qs3_debug_pair_spans(uint64_t* out, uint32_t capacity)
{
    using namespace qs3;
    if (out == nullptr || capacity < kTraceClusters * 3)
        return QSFI_STATUS_INVALID_ARGUMENT;
    if (cudaDeviceSynchronize() != cudaSuccess
        || cudaMemcpyFromSymbol(out, g_pair_spans, kTraceClusters * 3 * sizeof(uint64_t)) != cudaSuccess)
        return QSFI_STATUS_CUDA_ERROR;
    return QSFI_STATUS_OK;
}
