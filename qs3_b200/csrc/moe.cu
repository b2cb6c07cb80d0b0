// MoE entry points of the C ABI: plan, workspace sizing, routed-expert execution in
// bf16 and NVFP4, and the whole-layer call. The op sequence is upstream's
// (qsfi_moe.cu:539-724 and src/model.rs:2072-2228) with the element-wise steps
// folded into GEMM epilogues and one combine kernel.
#include "common.cuh"
#include "nvfp4.cuh"

#include <algorithm>
#include <cmath>
#include <limits>
#include <new>

namespace qs3 {

cudaError_t launch_tile_scales(const uint8_t* linear, uint32_t experts, uint32_t rows, uint32_t k,
                               int gated, uint8_t* tiled, cudaStream_t stream);

namespace {

template <typename T> T* carve(char* base, size_t& offset, size_t count)
{
    offset = align_up(offset, kWorkspaceAlign);
    T* p = base != nullptr ? reinterpret_cast<T*>(base + offset) : nullptr;
    offset += count * sizeof(T);
    return p;
}

bool mul_overflows(size_t a, size_t b, size_t* out)
{
    if (a != 0 && b > std::numeric_limits<size_t>::max() / a)
        return true;
    *out = a * b;
    return false;
}

// Size upstream's staged bf16 backend asks for (qsfi_moe.cu:67-121). The upstream
// Rust caller re-derives this number and refuses a smaller workspace
// (src/ffi/qsfi.rs:472-516,539-587), so the size reported here is never below it.
bool upstream_bf16_workspace_bytes(const qsfi_moe_plan_desc& d, uint32_t num_tokens, size_t* out)
{
    size_t routes = 0, hidden = 0, gate_up = 0, act = 0, twice_i = 0;
    if (mul_overflows(num_tokens, d.top_k, &routes) || mul_overflows(routes, d.hidden_size, &hidden)
        || mul_overflows(d.intermediate_size, 2, &twice_i) || mul_overflows(routes, twice_i, &gate_up)
        || mul_overflows(routes, d.intermediate_size, &act))
        return false;
    const size_t e = d.local_num_experts;
    size_t off = 0;
    const auto take = [&off](size_t count, size_t elem) {
        off = align_up(off, kWorkspaceAlign);
        off += count * elem;
    };
    take(e, 4);          // counts
    take(e + 1, 4);      // indptr
    take(e, 4);          // write_offsets
    take(routes, 4);     // route_rows
    take(routes, 4);     // row_tokens
    take(routes, 4);     // row_scales
    take(hidden, 2);     // expanded_hidden
    take(gate_up, 2);    // gemm1_out
    take(act, 2);        // act
    take(hidden, 2);     // gemm2_out
    take(e * 3, 4);      // problems
    for (int i = 0; i < 6; ++i)
        take(e, 8);      // x/w/y pointers and leading dimensions
    *out = align_up(off, kWorkspaceAlign);
    return true;
}

// ---- workspace layouts of this build ---------------------------------------------------

struct Bf16Workspace {
    RouteTables rt;
    __nv_bfloat16* expanded; // [pad_rows, H]
    __nv_bfloat16* act;      // [pad_rows, I]
    __nv_bfloat16* y2;       // [pad_rows, H]
    size_t bytes;
};

Bf16Workspace carve_bf16(char* base, const qsfi_moe_plan_desc& d, uint32_t num_tokens)
{
    Bf16Workspace w {};
    const uint32_t routes = num_tokens * d.top_k;
    size_t off = route_tables_carve(base, routes, d.local_num_experts, &w.rt);
    const size_t rows = w.rt.max_pad_rows;
    w.expanded = carve<__nv_bfloat16>(base, off, rows * d.hidden_size);
    w.act = carve<__nv_bfloat16>(base, off, rows * d.intermediate_size);
    w.y2 = carve<__nv_bfloat16>(base, off, rows * d.hidden_size);
    w.bytes = align_up(off, kWorkspaceAlign);
    return w;
}

struct Nvfp4Workspace {
    RouteTables rt;
    uint8_t* xq;       // [pad_rows, H/2]
    uint8_t* xq_sf;    // tiled(pad_rows, H)
    uint8_t* act;      // [pad_rows, I/2]
    uint8_t* act_sf;   // tiled(pad_rows, I)
    __nv_bfloat16* y2; // [pad_rows, H]
    uint8_t* gu_sf;    // per-call re-tiled weight scales (declared-ABI entry only)
    uint8_t* d_sf;
    size_t bytes;
};

Nvfp4Workspace carve_nvfp4(char* base, const qsfi_moe_plan_desc& d, uint32_t num_tokens, bool retile)
{
    Nvfp4Workspace w {};
    const uint32_t routes = num_tokens * d.top_k;
    size_t off = route_tables_carve(base, routes, d.local_num_experts, &w.rt,
                                    nvfp4_tile_rows(routes, d.local_num_experts, d.hidden_size, d.intermediate_size));
    const size_t rows = w.rt.max_pad_rows;
    const size_t h = d.hidden_size, i = d.intermediate_size, e = d.local_num_experts;
    w.xq = carve<uint8_t>(base, off, rows * h / 2);
    w.xq_sf = carve<uint8_t>(base, off, qs3_nvfp4_tiled_scale_bytes(rows, h));
    w.act = carve<uint8_t>(base, off, rows * i / 2);
    w.act_sf = carve<uint8_t>(base, off, qs3_nvfp4_tiled_scale_bytes(rows, i));
    w.y2 = carve<__nv_bfloat16>(base, off, rows * h);
    if (retile) {
        w.gu_sf = carve<uint8_t>(base, off, e * qs3_nvfp4_tiled_scale_bytes(2 * i, h));
        w.d_sf = carve<uint8_t>(base, off, e * qs3_nvfp4_tiled_scale_bytes(h, i));
    }
    w.bytes = align_up(off, kWorkspaceAlign);
    return w;
}

bool is_fp8_plan(const qsfi_moe_plan_desc& d)
{
    return static_cast<int>(d.backend) == QS3_MOE_BACKEND_FP8_BLOCKSCALE;
}

struct Fp8Workspace {
    RouteTables rt;    // token tiles of fp8_tile_rows rows
    uint8_t* xq;       // [pad_rows, H] e4m3
    float* xq_s;       // [pad_rows, H/128]
    uint8_t* act;      // [pad_rows, I] e4m3
    float* act_s;      // [pad_rows, I/128]
    __nv_bfloat16* y2; // [pad_rows, H]
    size_t bytes;
};

Fp8Workspace carve_fp8(char* base, const qsfi_moe_plan_desc& d, uint32_t num_tokens)
{
    Fp8Workspace w {};
    const uint32_t routes = num_tokens * d.top_k;
    size_t off = route_tables_carve(base, routes, d.local_num_experts, &w.rt,
                                    fp8_tile_rows(routes, d.local_num_experts));
    const size_t rows = w.rt.max_pad_rows;
    const size_t h = d.hidden_size, i = d.intermediate_size;
    w.xq = carve<uint8_t>(base, off, rows * h);
    w.xq_s = carve<float>(base, off, rows * (h / 128));
    w.act = carve<uint8_t>(base, off, rows * i);
    w.act_s = carve<float>(base, off, rows * (i / 128));
    w.y2 = carve<__nv_bfloat16>(base, off, rows * h);
    w.bytes = align_up(off, kWorkspaceAlign);
    return w;
}

// Extra buffers of the whole-layer call, carved after the routed-expert workspace.
struct LayerExtra {
    float* logits;          // [T, E]
    int32_t* topk_ids;      // [T, K]
    float* topk_weights;    // [T, K]
    __nv_bfloat16* sh_act;  // bf16 plans: [T, Is]
    __nv_bfloat16* sh_out;  // [T, H]
    uint8_t* sh_xq;         // NVFP4 plans: hidden quantised in token order [T128, H/2]
    uint8_t* sh_xq_sf;
    uint8_t* sh_actq;       // [T128, Is/2]
    uint8_t* sh_actq_sf;
    size_t bytes;
};

LayerExtra carve_layer(char* base, size_t start, const qsfi_moe_plan_desc& d, uint32_t num_tokens,
                       uint32_t shared_inter, bool nvfp4)
{
    LayerExtra x {};
    size_t off = start;
    const size_t t = num_tokens, h = d.hidden_size;
    x.logits = carve<float>(base, off, t * d.num_experts);
    x.topk_ids = carve<int32_t>(base, off, t * d.top_k);
    x.topk_weights = carve<float>(base, off, t * d.top_k);
    if (nvfp4) {
        // tokens quantised once, in token order: source of the routed gather and A operand
        // of the shared expert
        const size_t t128 = align_up(t, kTileM);
        x.sh_xq = carve<uint8_t>(base, off, t128 * h / 2);
        x.sh_xq_sf = carve<uint8_t>(base, off, qs3_nvfp4_tiled_scale_bytes(t128, h));
    }
    if (shared_inter != 0) {
        x.sh_out = carve<__nv_bfloat16>(base, off, t * h);
        if (nvfp4) {
            const size_t t128 = align_up(t, kTileM);
            x.sh_actq = carve<uint8_t>(base, off, t128 * shared_inter / 2);
            x.sh_actq_sf = carve<uint8_t>(base, off, qs3_nvfp4_tiled_scale_bytes(t128, shared_inter));
        } else {
            x.sh_act = carve<__nv_bfloat16>(base, off, t * shared_inter);
        }
    }
    x.bytes = align_up(off, kWorkspaceAlign);
    return x;
}

// ---- validation ------------------------------------------------------------------------

// Same checks and messages as upstream qsfi_validate_native_tensor
// (qsfi_native_common.h:29-55).
template <typename Tensor>
qsfi_status validate_tensor(qsfi_context* ctx, const Tensor& t, const char* name, qsfi_dtype dtype)
{
    if (t.data == nullptr)
        return set_invalid_arg(ctx, "%s.data must not be null", name);
    if (t.dtype != dtype)
        return set_invalid_arg(ctx, "%s dtype does not match expected dtype", name);
    constexpr uint32_t rank = sizeof(t.shape) / sizeof(t.shape[0]);
    for (uint32_t i = 0; i < rank; ++i)
        if (t.shape[i] <= 0 || t.stride[i] <= 0)
            return set_invalid_arg(ctx, "%s shape/stride entries must be positive", name);
    return QSFI_STATUS_OK;
}

qsfi_status not_contiguous(qsfi_context* ctx, const char* name)
{
    return set_invalid_arg(ctx, "%s must be contiguous in qsfi MoE staged BF16 backend", name);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// upstream validate_plan_desc, qsfi_moe.cu:144-200, minus the two rejections this
// build lifts (partial local expert range; see include/qs3_moe.h).
qsfi_status validate_plan_desc(qsfi_context* ctx, const qsfi_moe_plan_desc* d)
{
    if (d == nullptr)
        return set_invalid_arg(ctx, "desc is null");
    if (d->max_num_tokens == 0 || d->hidden_size == 0 || d->intermediate_size == 0
        || d->num_experts == 0 || d->top_k == 0 || d->local_num_experts == 0)
        return set_invalid_arg(ctx, "MoE plan dimensions must be non-zero");
    if (static_cast<uint64_t>(d->local_expert_offset) + d->local_num_experts > d->num_experts)
        return set_invalid_arg(ctx, "MoE local expert range exceeds num_experts");
    if (d->route_mode != QSFI_MOE_ROUTE_PRECOMPUTED_TOPK && d->route_mode != QSFI_MOE_ROUTE_ROUTER_LOGITS)
        return set_unsupported(ctx, "unsupported MoE route mode");
    if (d->top_k > 32)
        return set_unsupported(ctx, "MoE top_k above 32 is not supported");
    if (d->local_num_experts > 8192)
        return set_unsupported(ctx, "more than 8192 local experts are not supported");
    if (d->backend == QSFI_MOE_BACKEND_FLASHINFER_STAGED_BF16) {
        if (d->activation_dtype != QSFI_DTYPE_BF16 || d->weight_dtype != QSFI_DTYPE_BF16
            || d->output_dtype != QSFI_DTYPE_BF16)
            return set_invalid_arg(ctx, "staged BF16 MoE requires bf16 activation, weight, and output dtypes");
        if (d->hidden_size % 8 != 0 || d->intermediate_size % 8 != 0)
            return set_invalid_arg(ctx, "staged BF16 MoE requires hidden_size and intermediate_size divisible by 8");
        return QSFI_STATUS_OK;
    }
    if (d->backend == QSFI_MOE_BACKEND_FLASHINFER_NVFP4) {
        if (d->activation_dtype != QSFI_DTYPE_NVFP4_E2M1 || d->weight_dtype != QSFI_DTYPE_NVFP4_E2M1
            || d->output_dtype != QSFI_DTYPE_BF16)
            return set_invalid_arg(ctx, "NVFP4 MoE plan requires nvfp4 activation/weight and bf16 output dtypes");
        if (d->hidden_size % 16 != 0 || d->intermediate_size % 16 != 0)
            return set_invalid_arg(ctx, "NVFP4 MoE requires hidden_size and intermediate_size divisible by 16");
        return QSFI_STATUS_OK;
    }
    if (is_fp8_plan(*d)) {
        if (d->activation_dtype != QSFI_DTYPE_FP8_E4M3 || d->weight_dtype != QSFI_DTYPE_FP8_E4M3
            || d->output_dtype != QSFI_DTYPE_BF16)
            return set_invalid_arg(ctx, "FP8 MoE plan requires fp8_e4m3 activation/weight and bf16 output dtypes");
        if (d->hidden_size % 128 != 0 || d->intermediate_size % 128 != 0)
            return set_invalid_arg(ctx, "FP8 MoE requires hidden_size and intermediate_size divisible by 128");
        if (d->hidden_size > 4096 || d->intermediate_size > 4096)
            return set_unsupported(ctx, "FP8 MoE supports hidden_size and intermediate_size up to 4096");
        return QSFI_STATUS_OK;
    }
    return set_unsupported(ctx, "unsupported MoE backend");
}

// upstream validate_moe_launch_limits, qsfi_moe.cu:202-226
qsfi_status validate_limits(qsfi_context* ctx, const qsfi_moe_plan_desc& p, uint32_t num_tokens)
{
    const uint64_t routes = static_cast<uint64_t>(num_tokens) * p.top_k;
    const uint64_t i32max = static_cast<uint64_t>(std::numeric_limits<int32_t>::max());
    if (routes + static_cast<uint64_t>(p.local_num_experts) * kTileM + kTileM > i32max)
        return set_unsupported(ctx, "MoE route count exceeds int32 grouped-GEMM limits");
    if (p.hidden_size > i32max || 2ull * p.intermediate_size > i32max)
        return set_unsupported(ctx, "MoE dimensions exceed int32 grouped-GEMM limits");
    RouteTables rt {};
    route_tables_carve(nullptr, static_cast<uint32_t>(routes), p.local_num_experts, &rt,
                       is_fp8_plan(p) ? fp8_tile_rows(static_cast<uint32_t>(routes), p.local_num_experts)
                                      : static_cast<uint32_t>(kTileM));
    if (rt.max_tiles > 65535)
        return set_unsupported(ctx, "MoE launch grid is too large");
    return QSFI_STATUS_OK;
}

// NVFP4 tensor-core path needs whole scale tiles along k and along the gate rows.
qsfi_status validate_nvfp4_dims(qsfi_context* ctx, uint32_t hidden, uint32_t inter, const char* what)
{
    if (hidden % 256 != 0 || inter % 256 != 0)
        return set_unsupported(ctx, "NVFP4 MoE execution requires %s hidden and intermediate sizes divisible by 256", what);
    return QSFI_STATUS_OK;
}

// ---- routed experts ----------------------------------------------------------------------

GemmProblem grouped_problem(const RouteTables& rt, uint32_t groups)
{
    GemmProblem g {};
    g.a_rows = rt.max_pad_rows;
    g.groups = groups;
    g.tile_expert = rt.tile_expert;
    g.tile_row0 = rt.tile_row0;
    g.tile_nrows = rt.tile_nrows;
    g.total_tiles = rt.total_tiles;
    g.max_tiles = rt.max_tiles;
    g.tile_rows = rt.tile_rows;
    g.pair_expert = rt.pair_expert;
    g.pair_row0 = rt.pair_row0;
    g.pair_nrows = rt.pair_nrows;
    g.pair_counts = rt.pair_counts;
    return g;
}

qsfi_status gemm_on_stream(qsfi_context* ctx, const GemmProblem& g, const char* op, cudaStream_t stream)
{
    const char* why = nullptr;
    cudaError_t err = launch_gemm(g, stream, &why);
    if (err == cudaErrorNotSupported && why != nullptr)
        return set_unsupported(ctx, "%s: %s", op, why);
    if (err != cudaSuccess && why != nullptr)
        return set_error(ctx, QSFI_STATUS_BACKEND_ERROR, QSFI_ERROR_SOURCE_QSFI, static_cast<int32_t>(err),
                         "%s: %s", op, why);
    return set_cuda_error(ctx, err, op);
}

qsfi_status gemm_or_error(qsfi_context* ctx, const GemmProblem& g, const char* op)
{
    return gemm_on_stream(ctx, g, op, ctx->stream);
}

// Side stream and events of a plan (see qsfi_moe_plan); false when they cannot be had, in
// which case the layer runs on the context's stream alone.
bool plan_side_stream(const qsfi_moe_plan* plan)
{
    if (plan->side_state == 0) {
        plan->side_state = -1;
        if (cudaStreamCreateWithFlags(&plan->side_stream, cudaStreamNonBlocking) == cudaSuccess
            && cudaEventCreateWithFlags(&plan->ev_fork, cudaEventDisableTiming) == cudaSuccess
            && cudaEventCreateWithFlags(&plan->ev_quant, cudaEventDisableTiming) == cudaSuccess
            && cudaEventCreateWithFlags(&plan->ev_shared, cudaEventDisableTiming) == cudaSuccess)
            plan->side_state = 1;
        else
            cudaGetLastError();
    }
    return plan->side_state == 1;
}

// Routed experts in bf16 on rows already described by `rt`:
// gather -> gate_up GEMM + SwiGLU -> down GEMM. Leaves Y2 in w.y2.
qsfi_status run_routed_bf16(qsfi_context* ctx, const qsfi_moe_plan_desc& p, const Bf16Workspace& w,
                            const __nv_bfloat16* hidden, uint32_t num_tokens,
                            const __nv_bfloat16* gate_up, const __nv_bfloat16* down)
{
    const uint32_t routes = num_tokens * p.top_k;
    cudaError_t err = launch_gather_bf16(hidden, w.rt.route_prows, routes, p.top_k, p.hidden_size,
                                         w.expanded, ctx->stream);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "MoE gather");
    stage_mark(ctx->stream, STAGE_GATE_UP_GEMM);
    GemmProblem g1 = grouped_problem(w.rt, p.local_num_experts);
    g1.a = w.expanded;
    g1.a_pitch_bytes = static_cast<uint64_t>(p.hidden_size) * 2;
    g1.b = gate_up;
    g1.b_pitch_bytes = static_cast<uint64_t>(p.hidden_size) * 2;
    g1.n = p.intermediate_size;
    g1.k = p.hidden_size;
    g1.gated = 1;
    g1.epilogue = EPI_SWIGLU_BF16;
    g1.out = w.act;
    g1.out_pitch_elems = p.intermediate_size;
    qsfi_status status = gemm_or_error(ctx, g1, "MoE gate_up GEMM");
    if (status != QSFI_STATUS_OK)
        return status;
    stage_mark(ctx->stream, STAGE_DOWN_GEMM);
    GemmProblem g2 = grouped_problem(w.rt, p.local_num_experts);
    g2.a = w.act;
    g2.a_pitch_bytes = static_cast<uint64_t>(p.intermediate_size) * 2;
    g2.b = down;
    g2.b_pitch_bytes = static_cast<uint64_t>(p.intermediate_size) * 2;
    g2.n = p.hidden_size;
    g2.k = p.intermediate_size;
    g2.epilogue = EPI_STORE_BF16;
    g2.out = w.y2;
    g2.out_pitch_elems = p.hidden_size;
    return gemm_or_error(ctx, g2, "MoE down GEMM");
}

// Global scales of a gate_up weight: f32 [groups] (one per expert, gate and up rows alike) or
// f32 [2 * groups] (the gate-row scales followed by the up-row scales, as checkpoints that
// quantise gate_proj and up_proj separately have them).
bool gate_up_global_ok(const qsfi_tensor1& g, int64_t groups)
{
    return g.data == nullptr
        || (g.dtype == QSFI_DTYPE_F32 && (g.shape[0] == groups || g.shape[0] == 2 * groups) && g.stride[0] == 1);
}
const float* gate_up_global_up(const qsfi_tensor1& g, int64_t groups)
{
    return g.data != nullptr && g.shape[0] == 2 * groups ? static_cast<const float*>(g.data) + groups : nullptr;
}

struct Nvfp4Weights {
    const uint8_t* gu_packed;
    const uint8_t* gu_sf_tiled;
    const float* gu_global; // optional
    const float* gu_global_up; // optional: separate global scale of the up rows
    const uint8_t* d_packed;
    const uint8_t* d_sf_tiled;
    const float* d_global;  // optional
};

// Routed experts on NVFP4 operands; activation rows are already in w.xq / w.xq_sf.
qsfi_status run_routed_nvfp4(qsfi_context* ctx, const qsfi_moe_plan_desc& p, const Nvfp4Workspace& w,
                             const Nvfp4Weights& wt, float act_global, float act2_global)
{
    const float ga = act_global == 0.0f ? 1.0f : act_global;
    const float ga2 = act2_global == 0.0f ? 1.0f : act2_global;
    stage_mark(ctx->stream, STAGE_GATE_UP_GEMM);
    const uint32_t routes_hint = static_cast<uint32_t>(w.rt.max_pad_rows); // upper bound of the padded rows
    const uint32_t est_tiles = std::min<uint32_t>(w.rt.max_tiles,
                                                  p.local_num_experts + routes_hint / w.rt.tile_rows);
    GemmProblem g1 = grouped_problem(w.rt, p.local_num_experts);
    g1.est_tiles = est_tiles;
    g1.nvfp4 = 1;
    g1.a = w.xq;
    g1.a_pitch_bytes = p.hidden_size / 2;
    g1.a_scale_tiled = w.xq_sf;
    g1.b = wt.gu_packed;
    g1.b_pitch_bytes = p.hidden_size / 2;
    g1.b_scale_tiled = wt.gu_sf_tiled;
    g1.n = p.intermediate_size;
    g1.k = p.hidden_size;
    g1.gated = 1;
    g1.epilogue = EPI_SWIGLU_NVFP4;
    g1.out = w.act;
    g1.out_pitch_elems = p.intermediate_size / 2;
    g1.out_scale_tiled = w.act_sf;
    g1.alpha = ga;
    g1.group_scale = wt.gu_global;
    g1.group_scale_up = wt.gu_global_up;
    g1.out_global_scale = ga2;
    qsfi_status status = gemm_or_error(ctx, g1, "NVFP4 MoE gate_up GEMM");
    if (status != QSFI_STATUS_OK)
        return status;
    stage_mark(ctx->stream, STAGE_DOWN_GEMM);
    GemmProblem g2 = grouped_problem(w.rt, p.local_num_experts);
    g2.est_tiles = est_tiles;
    g2.nvfp4 = 1;
    g2.a = w.act;
    g2.a_pitch_bytes = p.intermediate_size / 2;
    g2.a_scale_tiled = w.act_sf;
    g2.b = wt.d_packed;
    g2.b_pitch_bytes = p.intermediate_size / 2;
    g2.b_scale_tiled = wt.d_sf_tiled;
    g2.n = p.hidden_size;
    g2.k = p.intermediate_size;
    g2.epilogue = EPI_STORE_BF16;
    g2.out = w.y2;
    g2.out_pitch_elems = p.hidden_size;
    g2.alpha = ga2;
    g2.group_scale = wt.d_global;
    return gemm_or_error(ctx, g2, "NVFP4 MoE down GEMM");
}

// Routed experts on FP8 operands; activation rows are already in w.xq / w.xq_s.
qsfi_status run_routed_fp8(qsfi_context* ctx, const qsfi_moe_plan_desc& p, const Fp8Workspace& w,
                           uint32_t num_tokens, const uint8_t* gu, const float* gu_scale, const uint8_t* down,
                           const float* down_scale)
{
    const uint32_t routes = num_tokens * p.top_k;
    const auto run = [&](const Fp8Gemm& g, const char* op) {
        const char* why = nullptr;
        cudaError_t err = launch_fp8_gemm(g, ctx->stream, &why);
        if (err == cudaErrorNotSupported && why != nullptr)
            return set_unsupported(ctx, "%s: %s", op, why);
        if (err != cudaSuccess && why != nullptr)
            return set_error(ctx, QSFI_STATUS_BACKEND_ERROR, QSFI_ERROR_SOURCE_QSFI, static_cast<int32_t>(err),
                             "%s: %s", op, why);
        return set_cuda_error(ctx, err, op);
    };
    Fp8Gemm g {};
    g.x_rows = w.rt.max_pad_rows;
    g.groups = p.local_num_experts;
    g.tile_expert = w.rt.tile_expert;
    g.tile_row0 = w.rt.tile_row0;
    g.tile_nrows = w.rt.tile_nrows;
    g.total_tiles = w.rt.total_tiles;
    g.max_tiles = w.rt.max_tiles;
    g.tile_rows = w.rt.tile_rows;
    g.est_tiles = std::min(p.local_num_experts, routes) + routes / w.rt.tile_rows;
    stage_mark(ctx->stream, STAGE_GATE_UP_GEMM);
    Fp8Gemm g1 = g;
    g1.x = w.xq;
    g1.x_scale = w.xq_s;
    g1.w = gu;
    g1.w_scale = gu_scale;
    g1.n = p.intermediate_size;
    g1.k = p.hidden_size;
    g1.gated = 1;
    g1.out = w.act;
    g1.out_scale = w.act_s;
    qsfi_status status = run(g1, "FP8 MoE gate_up GEMM");
    if (status != QSFI_STATUS_OK)
        return status;
    stage_mark(ctx->stream, STAGE_DOWN_GEMM);
    Fp8Gemm g2 = g;
    g2.x = w.act;
    g2.x_scale = w.act_s;
    g2.w = down;
    g2.w_scale = down_scale;
    g2.n = p.hidden_size;
    g2.k = p.intermediate_size;
    g2.out = w.y2;
    return run(g2, "FP8 MoE down GEMM");
}

qsfi_status validate_routing_tensors(qsfi_context* ctx, const qsfi_moe_plan_desc& p, uint32_t num_tokens,
                                     const qsfi_tensor2& ids, const qsfi_tensor2& weights,
                                     const qsfi_tensor2& out)
{
    qsfi_status status = validate_tensor(ctx, ids, "topk_ids", QSFI_DTYPE_I32);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, weights, "topk_weights", QSFI_DTYPE_F32);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, out, "out", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!contiguous2(ids))
        return not_contiguous(ctx, "topk_ids");
    if (!contiguous2(weights))
        return not_contiguous(ctx, "topk_weights");
    if (!contiguous2(out))
        return not_contiguous(ctx, "out");
    if (ids.shape[0] != num_tokens || ids.shape[1] != p.top_k || weights.shape[0] != num_tokens
        || weights.shape[1] != p.top_k || out.shape[0] != num_tokens || out.shape[1] != p.hidden_size)
        return set_invalid_arg(ctx, "MoE token/top-k tensor shape mismatch");
    return QSFI_STATUS_OK;
}

#if QSFI_ENABLE_CHECKED_VALIDATION
// upstream validate_routes_kernel, qsfi_moe.cu:307-325, with one difference: a plan that
// owns only part of the experts (expert parallelism, rejected upstream) accepts every id of
// the global range, since routes to other ranks' experts are legal there
__global__ void validate_routes_kernel(const int32_t* topk_ids, const float* topk_weights, uint32_t total_routes,
                                       int32_t first_valid, int32_t num_valid, int* error)
{
    const uint32_t route = blockIdx.x * blockDim.x + threadIdx.x;
    if (route >= total_routes)
        return;
    const int32_t rel = topk_ids[route] - first_valid;
    if (rel < 0 || rel >= num_valid || !isfinite(topk_weights[route]))
        atomicExch(error, 1);
}
#endif

// Checked builds: every route must name a valid expert and carry a finite weight (upstream
// validate_moe_routes, qsfi_moe.cu:494-537; costs one stream sync). Release builds: no-op.
qsfi_status validate_routes_checked(qsfi_context* ctx, const qsfi_moe_plan_desc& p, const void* ids,
                                    const void* weights, uint32_t total_routes)
{
#if !QSFI_ENABLE_CHECKED_VALIDATION
    (void)ctx;
    (void)p;
    (void)ids;
    (void)weights;
    (void)total_routes;
    return QSFI_STATUS_OK;
#else
    cudaError_t err = cudaSuccess;
    int* flag = checked_flag_reset(ctx->stream, &err);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "cudaMemsetAsync MoE route validation flag");
    const bool whole = p.local_num_experts == p.num_experts;
    validate_routes_kernel<<<(total_routes + 255) / 256, 256, 0, ctx->stream>>>(
        static_cast<const int32_t*>(ids), static_cast<const float*>(weights), total_routes,
        whole ? static_cast<int32_t>(p.local_expert_offset) : 0,
        static_cast<int32_t>(whole ? p.local_num_experts : p.num_experts), flag);
    note_launch();
    err = cudaGetLastError();
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "launch MoE route validation");
    const bool bad = checked_flag_finish(ctx->stream, &err);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "copy MoE route validation flag");
    if (bad)
        return set_invalid_arg(ctx, "MoE routes must target local experts and weights must be finite");
    return QSFI_STATUS_OK;
#endif
}

qsfi_status validate_workspace(qsfi_context* ctx, const qsfi_tensor1& ws, size_t need)
{
    qsfi_status status = validate_tensor(ctx, ws, "workspace", ws.dtype);
    if (status != QSFI_STATUS_OK)
        return status;
    if (ws.dtype != QSFI_DTYPE_U8 && ws.dtype != QSFI_DTYPE_I8)
        return set_invalid_arg(ctx, "MoE workspace dtype must be u8 or i8");
    if (!contiguous1(ws))
        return not_contiguous(ctx, "workspace");
    if (static_cast<size_t>(ws.shape[0]) < need)
        return set_invalid_arg(ctx, "MoE workspace is too small");
    if ((reinterpret_cast<uintptr_t>(ws.data) & 255u) != 0)
        return set_invalid_arg(ctx, "MoE workspace must be 256-byte aligned");
    return QSFI_STATUS_OK;
}

} // namespace
} // namespace qs3

using namespace qs3;

extern "C" {

qsfi_status qsfi_moe_plan_create(qsfi_context* ctx, const qsfi_moe_plan_desc* desc, qsfi_moe_plan** out)
{
    if (out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    *out = nullptr;
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = validate_plan_desc(ctx, desc);
    if (status != QSFI_STATUS_OK)
        return status;
    qsfi_moe_plan* plan = new (std::nothrow) qsfi_moe_plan;
    if (plan == nullptr)
        return set_error(ctx, QSFI_STATUS_OUT_OF_MEMORY, QSFI_ERROR_SOURCE_QSFI, 0, "allocating MoE plan");
    plan->desc = *desc;
    *out = plan;
    return QSFI_STATUS_OK;
}

void qsfi_moe_plan_destroy(qsfi_moe_plan* plan)
{
    if (plan == nullptr)
        return;
    if (plan->ev_fork != nullptr)
        cudaEventDestroy(plan->ev_fork);
    if (plan->ev_quant != nullptr)
        cudaEventDestroy(plan->ev_quant);
    if (plan->ev_shared != nullptr)
        cudaEventDestroy(plan->ev_shared);
    if (plan->side_stream != nullptr)
        cudaStreamDestroy(plan->side_stream);
    delete plan;
}

qsfi_status qsfi_moe_workspace_size(qsfi_context* ctx, const qsfi_moe_plan* plan, uint32_t num_tokens,
                                    size_t* device_bytes)
{
    if (device_bytes == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    *device_bytes = 0;
    if (ctx == nullptr || plan == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    const qsfi_moe_plan_desc& p = plan->desc;
    if (num_tokens > p.max_num_tokens)
        return set_invalid_arg(ctx, "num_tokens exceeds qsfi_moe_plan_desc.max_num_tokens");
    if (static_cast<uint64_t>(num_tokens) * p.top_k > 0x7fffffffull)
        return set_invalid_arg(ctx, "MoE expanded route count overflows size_t");
    if (p.backend == QSFI_MOE_BACKEND_FLASHINFER_STAGED_BF16) {
        size_t upstream = 0;
        if (!upstream_bf16_workspace_bytes(p, num_tokens, &upstream))
            return set_invalid_arg(ctx, "MoE workspace element count overflows size_t");
        *device_bytes = std::max(upstream, carve_bf16(nullptr, p, num_tokens).bytes);
        return QSFI_STATUS_OK;
    }
    if (is_fp8_plan(p)) {
        *device_bytes = carve_fp8(nullptr, p, num_tokens).bytes;
        return QSFI_STATUS_OK;
    }
    *device_bytes = carve_nvfp4(nullptr, p, num_tokens, true).bytes;
    return QSFI_STATUS_OK;
}

qsfi_status qsfi_moe_execute_bf16(qsfi_context* ctx, const qsfi_moe_plan* plan,
                                  const qsfi_moe_bf16_execute_desc* desc)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    // validation order of upstream validate_bf16_execute, qsfi_moe.cu:228-305
    if (plan == nullptr || desc == nullptr)
        return set_invalid_arg(ctx, "plan/desc is null");
    const qsfi_moe_plan_desc& p = plan->desc;
    if (p.backend != QSFI_MOE_BACKEND_FLASHINFER_STAGED_BF16)
        return set_invalid_arg(ctx, "qsfi_moe_execute_bf16 requires a staged BF16 MoE plan");
    if (desc->num_tokens == 0 || desc->num_tokens > p.max_num_tokens)
        return set_invalid_arg(ctx, "invalid MoE num_tokens");
    status = validate_tensor(ctx, desc->hidden, "hidden", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->topk_ids, "topk_ids", QSFI_DTYPE_I32);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->topk_weights, "topk_weights", QSFI_DTYPE_F32);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->gate_up_weight, "gate_up_weight", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->down_weight, "down_weight", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->out, "out", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->workspace, "workspace", desc->workspace.dtype);
    if (status != QSFI_STATUS_OK)
        return status;
    if (desc->workspace.dtype != QSFI_DTYPE_U8 && desc->workspace.dtype != QSFI_DTYPE_I8)
        return set_invalid_arg(ctx, "MoE workspace dtype must be u8 or i8");
    if (!contiguous2(desc->hidden))
        return not_contiguous(ctx, "hidden");
    if (!contiguous2(desc->topk_ids))
        return not_contiguous(ctx, "topk_ids");
    if (!contiguous2(desc->topk_weights))
        return not_contiguous(ctx, "topk_weights");
    if (!contiguous3(desc->gate_up_weight))
        return not_contiguous(ctx, "gate_up_weight");
    if (!contiguous3(desc->down_weight))
        return not_contiguous(ctx, "down_weight");
    if (!contiguous2(desc->out))
        return not_contiguous(ctx, "out");
    if (!contiguous1(desc->workspace))
        return not_contiguous(ctx, "workspace");
    const int64_t t = desc->num_tokens;
    if (desc->hidden.shape[0] != t || desc->hidden.shape[1] != p.hidden_size
        || desc->topk_ids.shape[0] != t || desc->topk_ids.shape[1] != p.top_k
        || desc->topk_weights.shape[0] != t || desc->topk_weights.shape[1] != p.top_k
        || desc->out.shape[0] != t || desc->out.shape[1] != p.hidden_size)
        return set_invalid_arg(ctx, "MoE token/top-k tensor shape mismatch");
    if (desc->gate_up_weight.shape[0] != p.local_num_experts
        || desc->gate_up_weight.shape[1] != 2ll * p.intermediate_size
        || desc->gate_up_weight.shape[2] != p.hidden_size
        || desc->down_weight.shape[0] != p.local_num_experts
        || desc->down_weight.shape[1] != p.hidden_size
        || desc->down_weight.shape[2] != p.intermediate_size)
        return set_invalid_arg(ctx, "MoE expert weight shape mismatch");
    if (static_cast<uint64_t>(desc->num_tokens) * p.top_k > 0x7fffffffull)
        return set_invalid_arg(ctx, "MoE expanded route count overflows size_t");
    size_t need = 0;
    status = qsfi_moe_workspace_size(ctx, plan, desc->num_tokens, &need);
    if (status != QSFI_STATUS_OK)
        return status;
    if (static_cast<size_t>(desc->workspace.shape[0]) < need)
        return set_invalid_arg(ctx, "MoE workspace is too small");
    status = validate_limits(ctx, p, desc->num_tokens);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!aligned16(desc->hidden.data) || !aligned16(desc->out.data) || !aligned16(desc->gate_up_weight.data)
        || !aligned16(desc->down_weight.data) || (reinterpret_cast<uintptr_t>(desc->workspace.data) & 255u) != 0)
        return set_invalid_arg(ctx, "MoE tensors must be 16-byte aligned and the workspace 256-byte aligned");

    status = validate_routes_checked(ctx, p, desc->topk_ids.data, desc->topk_weights.data,
                                     desc->num_tokens * p.top_k);
    if (status != QSFI_STATUS_OK)
        return status;
    Bf16Workspace w = carve_bf16(static_cast<char*>(desc->workspace.data), p, desc->num_tokens);
    const uint32_t routes = desc->num_tokens * p.top_k;
    cudaError_t err = launch_route_sort(static_cast<const int32_t*>(desc->topk_ids.data),
                                        static_cast<const float*>(desc->topk_weights.data), routes, p.top_k,
                                        p.local_expert_offset, p.local_num_experts, w.rt, ctx->stream);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "MoE route sort");
    status = run_routed_bf16(ctx, p, w, static_cast<const __nv_bfloat16*>(desc->hidden.data), desc->num_tokens,
                             static_cast<const __nv_bfloat16*>(desc->gate_up_weight.data),
                             static_cast<const __nv_bfloat16*>(desc->down_weight.data));
    if (status != QSFI_STATUS_OK)
        return status;
    CombineParams cp {};
    cp.route_prows = w.rt.route_prows;
    cp.topk_weights = static_cast<const float*>(desc->topk_weights.data);
    cp.expert_out = w.y2;
    cp.out = static_cast<__nv_bfloat16*>(desc->out.data);
    cp.num_tokens = desc->num_tokens;
    cp.top_k = p.top_k;
    cp.hidden_size = p.hidden_size;
    return set_cuda_error(ctx, launch_combine(cp, ctx->stream), "qsfi_moe_execute_bf16");
}

qsfi_status qsfi_moe_execute_nvfp4(qsfi_context* ctx, const qsfi_moe_plan* plan,
                                   const qsfi_moe_nvfp4_execute_desc* desc)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    if (plan == nullptr || desc == nullptr)
        return set_invalid_arg(ctx, "plan/desc is null");
    const qsfi_moe_plan_desc& p = plan->desc;
    if (p.backend != QSFI_MOE_BACKEND_FLASHINFER_NVFP4)
        return set_invalid_arg(ctx, "qsfi_moe_execute_nvfp4 requires an NVFP4 MoE plan");
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (desc->num_tokens == 0 || desc->num_tokens > p.max_num_tokens)
        return set_invalid_arg(ctx, "invalid MoE num_tokens");
    const int64_t t = desc->num_tokens, h = p.hidden_size, i = p.intermediate_size, e = p.local_num_experts;
    status = validate_tensor(ctx, desc->hidden_packed, "hidden_packed", QSFI_DTYPE_U8);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->hidden_scale, "hidden_scale", QSFI_DTYPE_FP8_E4M3);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->gate_up_weight_packed, "gate_up_weight_packed", QSFI_DTYPE_U8);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->gate_up_weight_scale, "gate_up_weight_scale", QSFI_DTYPE_FP8_E4M3);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->down_weight_packed, "down_weight_packed", QSFI_DTYPE_U8);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->down_weight_scale, "down_weight_scale", QSFI_DTYPE_FP8_E4M3);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_routing_tensors(ctx, p, desc->num_tokens, desc->topk_ids, desc->topk_weights, desc->out);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!contiguous2(desc->hidden_packed) || !contiguous2(desc->hidden_scale)
        || !contiguous3(desc->gate_up_weight_packed) || !contiguous3(desc->gate_up_weight_scale)
        || !contiguous3(desc->down_weight_packed) || !contiguous3(desc->down_weight_scale))
        return set_invalid_arg(ctx, "NVFP4 MoE tensors must be contiguous");
    // declared shapes, upstream qsfi.h:249-266
    if (desc->hidden_packed.shape[0] != t || desc->hidden_packed.shape[1] != h / 2
        || desc->hidden_scale.shape[0] != t || desc->hidden_scale.shape[1] != h / 16)
        return set_invalid_arg(ctx, "NVFP4 MoE hidden tensor shape mismatch");
    if (desc->gate_up_weight_packed.shape[0] != e || desc->gate_up_weight_packed.shape[1] != 2 * i
        || desc->gate_up_weight_packed.shape[2] != h / 2 || desc->gate_up_weight_scale.shape[0] != e
        || desc->gate_up_weight_scale.shape[1] != 2 * i || desc->gate_up_weight_scale.shape[2] != h / 16
        || desc->down_weight_packed.shape[0] != e || desc->down_weight_packed.shape[1] != h
        || desc->down_weight_packed.shape[2] != i / 2 || desc->down_weight_scale.shape[0] != e
        || desc->down_weight_scale.shape[1] != h || desc->down_weight_scale.shape[2] != i / 16)
        return set_invalid_arg(ctx, "NVFP4 MoE expert weight shape mismatch");
    if (desc->expert_output_scale.data != nullptr
        && (desc->expert_output_scale.dtype != QSFI_DTYPE_F32 || desc->expert_output_scale.shape[0] != e
            || !contiguous1(desc->expert_output_scale)))
        return set_invalid_arg(ctx, "expert_output_scale must be a contiguous f32 [local_num_experts] tensor");
    status = validate_nvfp4_dims(ctx, p.hidden_size, p.intermediate_size, "");
    if (status != QSFI_STATUS_OK)
        return status;
    size_t need = 0;
    status = qsfi_moe_workspace_size(ctx, plan, desc->num_tokens, &need);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_workspace(ctx, desc->workspace, need);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_limits(ctx, p, desc->num_tokens);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!aligned16(desc->hidden_packed.data) || !aligned16(desc->out.data)
        || !aligned16(desc->gate_up_weight_packed.data) || !aligned16(desc->down_weight_packed.data)
        || (reinterpret_cast<uintptr_t>(desc->hidden_scale.data) & 3u) != 0
        || (reinterpret_cast<uintptr_t>(desc->gate_up_weight_scale.data) & 3u) != 0
        || (reinterpret_cast<uintptr_t>(desc->down_weight_scale.data) & 3u) != 0)
        return set_invalid_arg(ctx, "NVFP4 MoE tensors must be 16-byte aligned (scales 4-byte aligned)");

    status = validate_routes_checked(ctx, p, desc->topk_ids.data, desc->topk_weights.data,
                                     desc->num_tokens * p.top_k);
    if (status != QSFI_STATUS_OK)
        return status;
    Nvfp4Workspace w = carve_nvfp4(static_cast<char*>(desc->workspace.data), p, desc->num_tokens, true);
    const uint32_t routes = desc->num_tokens * p.top_k;
    cudaStream_t st = ctx->stream;
    // The declared ABI carries row-major scales; the tensor-core path wants them
    // tiled. Re-tile the weight scales into the workspace (callers that prepare
    // weights once use qs3_moe_layer_execute, which takes tiled scales).
    cudaError_t err = launch_tile_scales(static_cast<const uint8_t*>(desc->gate_up_weight_scale.data),
                                         p.local_num_experts, 2 * p.intermediate_size, p.hidden_size, 1,
                                         w.gu_sf, st);
    if (err == cudaSuccess)
        err = launch_tile_scales(static_cast<const uint8_t*>(desc->down_weight_scale.data), p.local_num_experts,
                                 p.hidden_size, p.intermediate_size, 0, w.d_sf, st);
    if (err == cudaSuccess)
        err = launch_route_sort(static_cast<const int32_t*>(desc->topk_ids.data),
                                static_cast<const float*>(desc->topk_weights.data), routes, p.top_k,
                                p.local_expert_offset, p.local_num_experts, w.rt, st);
    if (err == cudaSuccess)
        err = launch_nvfp4_gather_tiles(static_cast<const uint8_t*>(desc->hidden_packed.data),
                                        static_cast<const uint8_t*>(desc->hidden_scale.data), w.rt, routes,
                                        p.top_k, p.hidden_size, w.xq, w.xq_sf, st);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "NVFP4 MoE routing");
    Nvfp4Weights wt {};
    wt.gu_packed = static_cast<const uint8_t*>(desc->gate_up_weight_packed.data);
    wt.gu_sf_tiled = w.gu_sf;
    wt.d_packed = static_cast<const uint8_t*>(desc->down_weight_packed.data);
    wt.d_sf_tiled = w.d_sf;
    wt.d_global = static_cast<const float*>(desc->expert_output_scale.data);
    status = run_routed_nvfp4(ctx, p, w, wt, 1.0f, 1.0f);
    if (status != QSFI_STATUS_OK)
        return status;
    CombineParams cp {};
    cp.route_prows = w.rt.route_prows;
    cp.topk_weights = static_cast<const float*>(desc->topk_weights.data);
    cp.expert_out = w.y2;
    cp.out = static_cast<__nv_bfloat16*>(desc->out.data);
    cp.num_tokens = desc->num_tokens;
    cp.top_k = p.top_k;
    cp.hidden_size = p.hidden_size;
    return set_cuda_error(ctx, launch_combine(cp, st), "qsfi_moe_execute_nvfp4");
}

qsfi_status qs3_moe_routing_tables(qsfi_context* ctx, const qsfi_moe_plan* plan, uint32_t num_tokens,
                                   qsfi_device_ptr workspace, qs3_moe_routing_view* out)
{
    if (ctx == nullptr || plan == nullptr || out == nullptr || workspace == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    if (num_tokens == 0 || num_tokens > plan->desc.max_num_tokens)
        return set_invalid_arg(ctx, "invalid MoE num_tokens");
    RouteTables rt {};
    route_tables_carve(static_cast<char*>(workspace), num_tokens * plan->desc.top_k,
                       plan->desc.local_num_experts, &rt);
    out->counts = rt.counts;
    out->indptr = rt.indptr;
    out->route_rows = rt.route_rows;
    out->row_tokens = rt.row_tokens;
    out->row_scales = rt.row_scales;
    return QSFI_STATUS_OK;
}

qsfi_status qs3_moe_layer_workspace_size(qsfi_context* ctx, const qsfi_moe_plan* plan, uint32_t num_tokens,
                                         uint32_t shared_intermediate_size, size_t* device_bytes)
{
    if (device_bytes == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    *device_bytes = 0;
    if (ctx == nullptr || plan == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    const qsfi_moe_plan_desc& p = plan->desc;
    if (num_tokens == 0 || num_tokens > p.max_num_tokens)
        return set_invalid_arg(ctx, "invalid MoE num_tokens");
    if (static_cast<uint64_t>(num_tokens) * p.top_k > 0x7fffffffull)
        return set_invalid_arg(ctx, "MoE expanded route count overflows size_t");
    const bool nvfp4 = p.backend == QSFI_MOE_BACKEND_FLASHINFER_NVFP4;
    const size_t base = is_fp8_plan(p) ? carve_fp8(nullptr, p, num_tokens).bytes
        : nvfp4                        ? carve_nvfp4(nullptr, p, num_tokens, false).bytes
                                       : carve_bf16(nullptr, p, num_tokens).bytes;
    *device_bytes = carve_layer(nullptr, base, p, num_tokens, shared_intermediate_size, nvfp4).bytes;
    return QSFI_STATUS_OK;
}

qsfi_status qs3_moe_layer_execute(qsfi_context* ctx, const qsfi_moe_plan* plan, const qs3_moe_layer_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (plan == nullptr || d == nullptr)
        return set_invalid_arg(ctx, "plan/desc is null");
    const qsfi_moe_plan_desc& p = plan->desc;
    const bool nvfp4 = p.backend == QSFI_MOE_BACKEND_FLASHINFER_NVFP4;
    const bool fp8 = is_fp8_plan(p);
    if (d->num_tokens == 0 || d->num_tokens > p.max_num_tokens)
        return set_invalid_arg(ctx, "invalid MoE num_tokens");
    const int64_t t = d->num_tokens, h = p.hidden_size, i = p.intermediate_size, e = p.local_num_experts;
    const uint32_t is = d->shared_intermediate_size;
    const bool shared = d->shared_gate_up_weight.data != nullptr;
    if (fp8 && shared)
        return set_unsupported(ctx, "FP8 MoE layer does not take a shared expert");

    status = validate_tensor(ctx, d->hidden, "hidden", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, d->router_weight, "router_weight", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, d->out, "out", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!contiguous2(d->hidden) || !contiguous2(d->router_weight) || !contiguous2(d->out))
        return set_invalid_arg(ctx, "MoE layer tensors must be contiguous");
    if (d->hidden.shape[0] != t || d->hidden.shape[1] != h || d->out.shape[0] != t || d->out.shape[1] != h
        || d->router_weight.shape[0] != p.num_experts || d->router_weight.shape[1] != h)
        return set_invalid_arg(ctx, "MoE token/top-k tensor shape mismatch");
    if (d->router_bias.data != nullptr
        && (d->router_bias.dtype != QSFI_DTYPE_F32 || d->router_bias.shape[0] != p.num_experts
            || !contiguous1(d->router_bias)))
        return set_invalid_arg(ctx, "router_bias must be a contiguous f32 [num_experts] tensor");
    if (p.top_k > 16 || p.num_experts > 4096 || p.top_k > p.num_experts)
        return set_unsupported(ctx, "router supports top_k <= 16 and num_experts <= 4096");
    if (d->score != QSCU_ROUTER_SCORE_SOFTMAX && d->score != QSCU_ROUTER_SCORE_SIGMOID)
        return set_unsupported(ctx, "unsupported router score");
    if (!std::isfinite(d->routed_scaling_factor) || d->routed_scaling_factor <= 0.0f)
        return set_invalid_arg(ctx, "routed_scaling_factor must be finite and positive");
    const qsfi_dtype wdt = nvfp4 ? QSFI_DTYPE_U8 : fp8 ? QSFI_DTYPE_FP8_E4M3 : QSFI_DTYPE_BF16;
    const int64_t kdiv = nvfp4 ? 2 : 1;
    status = validate_tensor(ctx, d->gate_up_weight, "gate_up_weight", wdt);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, d->down_weight, "down_weight", wdt);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!contiguous3(d->gate_up_weight) || !contiguous3(d->down_weight)
        || d->gate_up_weight.shape[0] != e || d->gate_up_weight.shape[1] != 2 * i
        || d->gate_up_weight.shape[2] != h / kdiv || d->down_weight.shape[0] != e
        || d->down_weight.shape[1] != h || d->down_weight.shape[2] != i / kdiv)
        return set_invalid_arg(ctx, "MoE expert weight shape mismatch");
    if (shared) {
        if (is == 0 || is % (nvfp4 ? 256 : 8) != 0)
            return set_invalid_arg(ctx, "invalid shared_intermediate_size");
        status = validate_tensor(ctx, d->shared_gate_up_weight, "shared_gate_up_weight", wdt);
        if (status != QSFI_STATUS_OK)
            return status;
        status = validate_tensor(ctx, d->shared_down_weight, "shared_down_weight", wdt);
        if (status != QSFI_STATUS_OK)
            return status;
        status = validate_tensor(ctx, d->shared_gate_weight, "shared_gate_weight", QSFI_DTYPE_BF16);
        if (status != QSFI_STATUS_OK)
            return status;
        if (!contiguous3(d->shared_gate_up_weight) || !contiguous3(d->shared_down_weight)
            || !contiguous2(d->shared_gate_weight) || d->shared_gate_up_weight.shape[0] != 1
            || d->shared_gate_up_weight.shape[1] != 2ll * is || d->shared_gate_up_weight.shape[2] != h / kdiv
            || d->shared_down_weight.shape[0] != 1 || d->shared_down_weight.shape[1] != h
            || d->shared_down_weight.shape[2] != is / kdiv || d->shared_gate_weight.shape[0] != 1
            || d->shared_gate_weight.shape[1] != h)
            return set_invalid_arg(ctx, "MoE shared expert weight shape mismatch");
    }
    if (nvfp4) {
        status = validate_nvfp4_dims(ctx, p.hidden_size, p.intermediate_size, "");
        if (status != QSFI_STATUS_OK)
            return status;
        if (d->gate_up_scale_tiled.data == nullptr || d->down_scale_tiled.data == nullptr
            || static_cast<uint64_t>(d->gate_up_scale_tiled.shape[0]) < e * qs3_nvfp4_tiled_scale_bytes(2 * i, h)
            || static_cast<uint64_t>(d->down_scale_tiled.shape[0]) < e * qs3_nvfp4_tiled_scale_bytes(h, i))
            return set_invalid_arg(ctx, "NVFP4 MoE layer needs tiled weight scales of the right size");
        if (!gate_up_global_ok(d->gate_up_global_scale, e)
            || (shared && !gate_up_global_ok(d->shared_gate_up_global_scale, 1)))
            return set_invalid_arg(ctx, "gate_up global scales must be contiguous f32 [groups] or [2 * groups] tensors");
        if (shared
            && (d->shared_gate_up_scale_tiled.data == nullptr || d->shared_down_scale_tiled.data == nullptr
                || static_cast<uint64_t>(d->shared_gate_up_scale_tiled.shape[0])
                    < qs3_nvfp4_tiled_scale_bytes(2 * is, h)
                || static_cast<uint64_t>(d->shared_down_scale_tiled.shape[0])
                    < qs3_nvfp4_tiled_scale_bytes(h, is)))
            return set_invalid_arg(ctx, "NVFP4 MoE layer needs tiled shared-expert scales of the right size");
    }
    if (fp8) {
        const uint64_t gu_scales = static_cast<uint64_t>(e) * (2 * i / 128) * (h / 128);
        const uint64_t d_scales = static_cast<uint64_t>(e) * (h / 128) * (i / 128);
        if (d->gate_up_scale_tiled.data == nullptr || d->down_scale_tiled.data == nullptr
            || d->gate_up_scale_tiled.dtype != QSFI_DTYPE_F32 || d->down_scale_tiled.dtype != QSFI_DTYPE_F32
            || static_cast<uint64_t>(d->gate_up_scale_tiled.shape[0]) < gu_scales
            || static_cast<uint64_t>(d->down_scale_tiled.shape[0]) < d_scales)
            return set_invalid_arg(ctx, "FP8 MoE layer needs f32 block scales of the right size");
    }
    size_t need = 0;
    status = qs3_moe_layer_workspace_size(ctx, plan, d->num_tokens, shared ? is : 0, &need);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_workspace(ctx, d->workspace, need);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_limits(ctx, p, d->num_tokens);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!aligned16(d->hidden.data) || !aligned16(d->out.data) || !aligned16(d->router_weight.data)
        || !aligned16(d->gate_up_weight.data) || !aligned16(d->down_weight.data)
        || (shared && (!aligned16(d->shared_gate_up_weight.data) || !aligned16(d->shared_down_weight.data)
                       || !aligned16(d->shared_gate_weight.data))))
        return set_invalid_arg(ctx, "MoE tensors must be 16-byte aligned");

    const bool prequant = nvfp4 && d->hidden_packed.data != nullptr;
    if (prequant) {
        if (d->hidden_packed.dtype != QSFI_DTYPE_U8 || !contiguous2(d->hidden_packed)
            || d->hidden_packed.shape[0] < t || d->hidden_packed.shape[1] != h / 2
            || !aligned16(d->hidden_packed.data) || d->hidden_scale_tiled.data == nullptr
            || static_cast<uint64_t>(d->hidden_scale_tiled.shape[0])
                < qs3_nvfp4_tiled_scale_bytes(static_cast<uint64_t>(t), static_cast<uint64_t>(h))
            || !aligned16(d->hidden_scale_tiled.data))
            return set_invalid_arg(ctx, "pre-quantised tokens need u8 [num_tokens, hidden/2] codes and tiled scales");
    }

    const bool post_norm = d->residual_inout.data != nullptr;
    if (post_norm) {
        if (d->residual_inout.dtype != QSFI_DTYPE_BF16 || !contiguous2(d->residual_inout)
            || d->residual_inout.shape[0] != t || d->residual_inout.shape[1] != h
            || d->next_norm_weight.data == nullptr || d->next_norm_weight.dtype != QSFI_DTYPE_BF16
            || d->next_norm_weight.shape[0] != h || !contiguous1(d->next_norm_weight)
            || !aligned16(d->residual_inout.data) || !aligned16(d->next_norm_weight.data))
            return set_invalid_arg(ctx, "fused post-MoE norm needs bf16 residual_inout [num_tokens, hidden] and "
                                        "next_norm_weight [hidden], 16-byte aligned");
        if (!std::isfinite(d->next_norm_eps) || d->next_norm_eps <= 0.0f)
            return set_invalid_arg(ctx, "rmsnorm eps must be finite and > 0");
        if (h > 2048)
            return set_unsupported(ctx, "fused post-MoE norm supports hidden_size up to 2048");
    }

    char* base = static_cast<char*>(d->workspace.data);
    cudaStream_t st = ctx->stream;
    const uint32_t routes = d->num_tokens * p.top_k;
    Bf16Workspace wb {};
    Nvfp4Workspace wn {};
    Fp8Workspace wf {};
    size_t routed_bytes = 0;
    if (fp8) {
        wf = carve_fp8(base, p, d->num_tokens);
        routed_bytes = wf.bytes;
    } else if (nvfp4) {
        wn = carve_nvfp4(base, p, d->num_tokens, false);
        routed_bytes = wn.bytes;
    } else {
        wb = carve_bf16(base, p, d->num_tokens);
        routed_bytes = wb.bytes;
    }
    const RouteTables& rt = fp8 ? wf.rt : nvfp4 ? wn.rt : wb.rt;
    LayerExtra x = carve_layer(base, routed_bytes, p, d->num_tokens, shared ? is : 0, nvfp4);
    const __nv_bfloat16* hidden = static_cast<const __nv_bfloat16*>(d->hidden.data);
    if (prequant) { // the caller's codes replace the layer's own token-order copy
        x.sh_xq = static_cast<uint8_t*>(d->hidden_packed.data);
        x.sh_xq_sf = static_cast<uint8_t*>(d->hidden_scale_tiled.data);
    }

    // NVFP4 shared expert as a dense problem over the tokens in natural order (A operand:
    // the tokens quantised once in x.sh_xq)
    const auto run_shared_nvfp4 = [&](cudaStream_t stream) -> qsfi_status {
        const float ga = d->act_global_scale == 0.0f ? 1.0f : d->act_global_scale;
        const float ga2 = d->act2_global_scale == 0.0f ? 1.0f : d->act2_global_scale;
        GemmProblem s1 {};
        s1.nvfp4 = 1;
        s1.a = x.sh_xq;
        s1.a_rows = d->num_tokens;
        s1.a_pitch_bytes = h / 2;
        s1.a_scale_tiled = x.sh_xq_sf;
        s1.b = d->shared_gate_up_weight.data;
        s1.b_pitch_bytes = h / 2;
        s1.b_scale_tiled = static_cast<const uint8_t*>(d->shared_gate_up_scale_tiled.data);
        s1.groups = 1;
        s1.n = is;
        s1.k = p.hidden_size;
        s1.gated = 1;
        s1.epilogue = EPI_SWIGLU_NVFP4;
        s1.out = x.sh_actq;
        s1.out_pitch_elems = is / 2;
        s1.out_scale_tiled = x.sh_actq_sf;
        s1.alpha = ga;
        s1.group_scale = static_cast<const float*>(d->shared_gate_up_global_scale.data);
        s1.group_scale_up = gate_up_global_up(d->shared_gate_up_global_scale, 1);
        s1.out_global_scale = ga2;
        qsfi_status st1 = gemm_on_stream(ctx, s1, "NVFP4 shared gate_up GEMM", stream);
        if (st1 != QSFI_STATUS_OK)
            return st1;
        GemmProblem s2 {};
        s2.nvfp4 = 1;
        s2.a = x.sh_actq;
        s2.a_rows = d->num_tokens;
        s2.a_pitch_bytes = is / 2;
        s2.a_scale_tiled = x.sh_actq_sf;
        s2.b = d->shared_down_weight.data;
        s2.b_pitch_bytes = is / 2;
        s2.b_scale_tiled = static_cast<const uint8_t*>(d->shared_down_scale_tiled.data);
        s2.groups = 1;
        s2.n = p.hidden_size;
        s2.k = is;
        s2.epilogue = EPI_STORE_BF16;
        s2.out = x.sh_out;
        s2.out_pitch_elems = p.hidden_size;
        s2.alpha = ga2;
        s2.group_scale = static_cast<const float*>(d->shared_down_global_scale.data);
        return gemm_on_stream(ctx, s2, "NVFP4 shared down GEMM", stream);
    };
    // With a shared expert, the token quantiser and the shared expert's two GEMMs depend on
    // the tokens only: they run on the plan's side stream beside the router chain (logits
    // GEMM, top-k, sort) and join the main stream where their results are consumed. The
    // per-stage recorder needs one timeline, so a profiled call stays on the main stream.
    const bool fork = nvfp4 && shared && !stage_recording() && plan_side_stream(plan);
    if (fork) {
        cudaStream_t side = plan->side_stream;
        cudaError_t ferr = cudaEventRecord(plan->ev_fork, st);
        if (ferr == cudaSuccess)
            ferr = cudaStreamWaitEvent(side, plan->ev_fork, 0);
        if (ferr == cudaSuccess && !prequant)
            ferr = launch_nvfp4_gather_quantize(hidden, nullptr, d->num_tokens, 1, p.hidden_size,
                                                d->act_global_scale, x.sh_xq, x.sh_xq_sf, side);
        if (ferr == cudaSuccess)
            ferr = cudaEventRecord(plan->ev_quant, side);
        if (ferr != cudaSuccess)
            return set_cuda_error(ctx, ferr, "NVFP4 MoE layer fork");
        status = run_shared_nvfp4(side);
        if (status != QSFI_STATUS_OK)
            return status;
        ferr = cudaEventRecord(plan->ev_shared, side);
        if (ferr != cudaSuccess)
            return set_cuda_error(ctx, ferr, "NVFP4 MoE layer fork");
    }

    stage_mark(st, STAGE_ROUTER_GEMM);
    // 1. router logits: f32 [T, E] = hidden . router_weight^T  (src/model.rs:2082-2090)
    float* logits = d->router_logits.data != nullptr ? static_cast<float*>(d->router_logits.data) : x.logits;
    GemmProblem gl {};
    gl.a = hidden;
    gl.a_rows = d->num_tokens;
    gl.a_pitch_bytes = static_cast<uint64_t>(h) * 2;
    gl.b = d->router_weight.data;
    gl.b_pitch_bytes = static_cast<uint64_t>(h) * 2;
    gl.groups = 1;
    gl.n = p.num_experts;
    gl.k = p.hidden_size;
    gl.epilogue = EPI_STORE_F32;
    gl.out = logits;
    gl.out_pitch_elems = p.num_experts;
    // split-k scratch for decode-sized batches: the routed experts' output buffer, which nothing touches
    // before the down projection (the side stream works on the shared expert's own buffers)
    {
        __nv_bfloat16* y2_buf = fp8 ? wf.y2 : nvfp4 ? wn.y2 : wb.y2;
        gl.splitk_scratch = reinterpret_cast<float*>(y2_buf);
        gl.splitk_scratch_bytes = static_cast<size_t>(rt.max_pad_rows) * p.hidden_size * sizeof(__nv_bfloat16);
    }
    status = gemm_or_error(ctx, gl, "MoE router-logits GEMM");
    if (status != QSFI_STATUS_OK)
        return status;

    stage_mark(st, STAGE_ROUTER_TOPK);
    // 2. top-k routing (src/model.rs:2092-2115)
    int32_t* ids = d->topk_ids.data != nullptr ? static_cast<int32_t*>(d->topk_ids.data) : x.topk_ids;
    float* wts = d->topk_weights.data != nullptr ? static_cast<float*>(d->topk_weights.data) : x.topk_weights;
    cudaError_t err = launch_router_topk(logits, 0, static_cast<const float*>(d->router_bias.data), ids, wts,
                                         d->num_tokens, p.num_experts, p.top_k,
                                         d->score == QSCU_ROUTER_SCORE_SIGMOID, d->renormalize != 0,
                                         d->routed_scaling_factor, st);
    // 3. permutation
    stage_mark(st, STAGE_ROUTE_SORT);
    if (err == cudaSuccess)
        err = launch_route_sort(ids, wts, routes, p.top_k, p.local_expert_offset, p.local_num_experts, rt, st);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "MoE routing");

    const __nv_bfloat16* y2 = nullptr;
    if (fp8) {
        // 4. quantise the routed rows straight from the bf16 tokens; 5./6. grouped GEMMs
        stage_mark(st, STAGE_GATHER);
        err = launch_fp8_gather_quantize(hidden, rt.route_prows, routes, p.top_k, p.hidden_size, wf.xq, wf.xq_s,
                                         st);
        if (err != cudaSuccess)
            return set_cuda_error(ctx, err, "FP8 MoE gather");
        status = run_routed_fp8(ctx, p, wf, d->num_tokens, static_cast<const uint8_t*>(d->gate_up_weight.data),
                                static_cast<const float*>(d->gate_up_scale_tiled.data),
                                static_cast<const uint8_t*>(d->down_weight.data),
                                static_cast<const float*>(d->down_scale_tiled.data));
        if (status != QSFI_STATUS_OK)
            return status;
        y2 = wf.y2;
    } else if (nvfp4) {
        // 4. quantise every token once (token order), then gather the codes by expert;
        //    5./6. grouped GEMMs
        stage_mark(st, STAGE_GATHER);
        if (fork)
            err = cudaStreamWaitEvent(st, plan->ev_quant, 0);
        else if (!prequant)
            err = launch_nvfp4_gather_quantize(hidden, nullptr, d->num_tokens, 1, p.hidden_size,
                                               d->act_global_scale, x.sh_xq, x.sh_xq_sf, st);
        if (err == cudaSuccess)
            err = launch_nvfp4_gather_tiles(x.sh_xq, x.sh_xq_sf, rt, routes, p.top_k, p.hidden_size, wn.xq, wn.xq_sf,
                                            st, 1);
        if (err != cudaSuccess)
            return set_cuda_error(ctx, err, "NVFP4 MoE gather");
        Nvfp4Weights wt {};
        wt.gu_packed = static_cast<const uint8_t*>(d->gate_up_weight.data);
        wt.gu_sf_tiled = static_cast<const uint8_t*>(d->gate_up_scale_tiled.data);
        wt.gu_global = static_cast<const float*>(d->gate_up_global_scale.data);
        wt.gu_global_up = gate_up_global_up(d->gate_up_global_scale, p.local_num_experts);
        wt.d_packed = static_cast<const uint8_t*>(d->down_weight.data);
        wt.d_sf_tiled = static_cast<const uint8_t*>(d->down_scale_tiled.data);
        wt.d_global = static_cast<const float*>(d->down_global_scale.data);
        status = run_routed_nvfp4(ctx, p, wn, wt, d->act_global_scale, d->act2_global_scale);
        if (status != QSFI_STATUS_OK)
            return status;
        y2 = wn.y2;
        if (shared) {
            // 7. shared expert
            stage_mark(st, STAGE_SHARED);
            if (fork) {
                err = cudaStreamWaitEvent(st, plan->ev_shared, 0);
                if (err != cudaSuccess)
                    return set_cuda_error(ctx, err, "NVFP4 MoE layer join");
            } else {
                status = run_shared_nvfp4(st);
                if (status != QSFI_STATUS_OK)
                    return status;
            }
        }
    } else {
        stage_mark(st, STAGE_GATHER);
        status = run_routed_bf16(ctx, p, wb, hidden, d->num_tokens,
                                 static_cast<const __nv_bfloat16*>(d->gate_up_weight.data),
                                 static_cast<const __nv_bfloat16*>(d->down_weight.data));
        if (status != QSFI_STATUS_OK)
            return status;
        y2 = wb.y2;
        if (shared) {
            // shared expert, src/model.rs:2174-2228, with SiLU*mul fused into the first GEMM
            stage_mark(st, STAGE_SHARED);
            GemmProblem s1 {};
            s1.a = hidden;
            s1.a_rows = d->num_tokens;
            s1.a_pitch_bytes = static_cast<uint64_t>(h) * 2;
            s1.b = d->shared_gate_up_weight.data;
            s1.b_pitch_bytes = static_cast<uint64_t>(h) * 2;
            s1.groups = 1;
            s1.n = is;
            s1.k = p.hidden_size;
            s1.gated = 1;
            s1.epilogue = EPI_SWIGLU_BF16;
            s1.out = x.sh_act;
            s1.out_pitch_elems = is;
            status = gemm_or_error(ctx, s1, "shared gate_up GEMM");
            if (status != QSFI_STATUS_OK)
                return status;
            GemmProblem s2 {};
            s2.a = x.sh_act;
            s2.a_rows = d->num_tokens;
            s2.a_pitch_bytes = static_cast<uint64_t>(is) * 2;
            s2.b = d->shared_down_weight.data;
            s2.b_pitch_bytes = static_cast<uint64_t>(is) * 2;
            s2.groups = 1;
            s2.n = p.hidden_size;
            s2.k = is;
            s2.epilogue = EPI_STORE_BF16;
            s2.out = x.sh_out;
            s2.out_pitch_elems = p.hidden_size;
            status = gemm_or_error(ctx, s2, "shared down GEMM");
            if (status != QSFI_STATUS_OK)
                return status;
        }
    }

    // 8. weighted combine (+ sigmoid-gated shared expert)
    stage_mark(st, STAGE_COMBINE);
    CombineParams cp {};
    cp.route_prows = rt.route_prows;
    cp.topk_weights = wts;
    cp.expert_out = y2;
    cp.out = static_cast<__nv_bfloat16*>(d->out.data);
    cp.num_tokens = d->num_tokens;
    cp.top_k = p.top_k;
    cp.hidden_size = p.hidden_size;
    if (shared) {
        cp.shared_out = x.sh_out;
        cp.hidden = hidden;
        cp.gate_w = static_cast<const __nv_bfloat16*>(d->shared_gate_weight.data);
        cp.round_before_shared = nvfp4 ? 0 : 1;
    }
    if (post_norm) {
        cp.residual = static_cast<__nv_bfloat16*>(d->residual_inout.data);
        cp.norm_weight = static_cast<const __nv_bfloat16*>(d->next_norm_weight.data);
        cp.norm_eps = d->next_norm_eps;
    }
    status = set_cuda_error(ctx, launch_combine(cp, st), "qs3_moe_layer_execute");
    stage_mark(st, STAGE_END);
    return status;
}

// ---- expert-parallel phases ------------------------------------------------------------
// One layer on n ranks = route (local tokens) -> token exchange -> local experts over the
// gathered tokens -> partial-sum exchange -> finish (shared expert + ordered sum). The
// exchanges are the caller's (NCCL); these three calls are the compute between them.

qsfi_status qs3_moe_ep_route(qsfi_context* ctx, const qsfi_moe_plan* plan, const qs3_moe_ep_route_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (plan == nullptr || d == nullptr)
        return set_invalid_arg(ctx, "plan/desc is null");
    const qsfi_moe_plan_desc& p = plan->desc;
    if (d->num_tokens == 0)
        return set_invalid_arg(ctx, "invalid MoE num_tokens");
    const int64_t t = d->num_tokens, h = p.hidden_size;
    const bool mapped = d->expert_id_map.data != nullptr;
    if (mapped
        && (d->expert_id_map.dtype != QSFI_DTYPE_I32 || !contiguous1(d->expert_id_map) || d->expert_id_map.shape[0] <= 0
            || d->dispatch_ids.data == nullptr || d->dispatch_ids.dtype != QSFI_DTYPE_I32
            || !contiguous2(d->dispatch_ids) || d->dispatch_ids.shape[0] != t || d->dispatch_ids.shape[1] != p.top_k))
        return set_invalid_arg(ctx, "expert_id_map must be a contiguous i32 [router experts] tensor with an i32 "
                                    "[num_tokens, top_k] dispatch_ids output");
    if (d->rank_mask.data != nullptr
        && (d->rank_mask.dtype != QSFI_DTYPE_I32 || !contiguous1(d->rank_mask) || d->rank_mask.shape[0] != t
            || d->num_ranks == 0 || d->num_ranks > 32))
        return set_invalid_arg(ctx, "rank_mask must be a contiguous i32 [num_tokens] tensor with 1..32 ranks");
    const int64_t router_experts = mapped ? d->expert_id_map.shape[0] : static_cast<int64_t>(p.num_experts);
    status = validate_tensor(ctx, d->hidden, "hidden", QSFI_DTYPE_BF16);
    if (status == QSFI_STATUS_OK)
        status = validate_tensor(ctx, d->router_weight, "router_weight", QSFI_DTYPE_BF16);
    if (status == QSFI_STATUS_OK)
        status = validate_tensor(ctx, d->router_logits, "router_logits", QSFI_DTYPE_F32);
    if (status == QSFI_STATUS_OK)
        status = validate_tensor(ctx, d->topk_ids, "topk_ids", QSFI_DTYPE_I32);
    if (status == QSFI_STATUS_OK)
        status = validate_tensor(ctx, d->topk_weights, "topk_weights", QSFI_DTYPE_F32);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!contiguous2(d->hidden) || !contiguous2(d->router_weight) || !contiguous2(d->router_logits)
        || !contiguous2(d->topk_ids) || !contiguous2(d->topk_weights))
        return set_invalid_arg(ctx, "MoE route tensors must be contiguous");
    if (d->hidden.shape[0] != t || d->hidden.shape[1] != h || d->router_weight.shape[0] != router_experts
        || d->router_weight.shape[1] != h || d->router_logits.shape[0] != t
        || d->router_logits.shape[1] != router_experts || d->topk_ids.shape[0] != t
        || d->topk_ids.shape[1] != p.top_k || d->topk_weights.shape[0] != t
        || d->topk_weights.shape[1] != p.top_k)
        return set_invalid_arg(ctx, "MoE token/top-k tensor shape mismatch");
    if (d->router_bias.data != nullptr
        && (d->router_bias.dtype != QSFI_DTYPE_F32 || d->router_bias.shape[0] != router_experts
            || !contiguous1(d->router_bias)))
        return set_invalid_arg(ctx, "router_bias must be a contiguous f32 [num_experts] tensor");
    if (p.top_k > 16 || router_experts > 4096 || p.top_k > router_experts)
        return set_unsupported(ctx, "router supports top_k <= 16 and num_experts <= 4096");
    if (!std::isfinite(d->routed_scaling_factor) || d->routed_scaling_factor <= 0.0f)
        return set_invalid_arg(ctx, "routed_scaling_factor must be finite and positive");
    const uint32_t num_router_experts = static_cast<uint32_t>(router_experts);
    const bool quantise = d->hidden_packed.data != nullptr;
    if (quantise) {
        if (h % 16 != 0 || d->hidden_packed.dtype != QSFI_DTYPE_U8 || !contiguous2(d->hidden_packed)
            || d->hidden_packed.shape[0] != t || d->hidden_packed.shape[1] != h / 2
            || d->hidden_scale.data == nullptr || d->hidden_scale.dtype != QSFI_DTYPE_FP8_E4M3
            || !contiguous2(d->hidden_scale) || d->hidden_scale.shape[0] != t
            || d->hidden_scale.shape[1] != h / 16)
            return set_invalid_arg(ctx, "NVFP4 MoE hidden tensor shape mismatch");
    }
    if (!aligned16(d->hidden.data) || !aligned16(d->router_weight.data)
        || (quantise && !aligned16(d->hidden_packed.data)))
        return set_invalid_arg(ctx, "MoE tensors must be 16-byte aligned");

    // The token quantiser depends on the tokens only: it runs on the plan's side stream beside the
    // router GEMM and the top-k and joins before the call returns its stream to the caller.
    qs3_nvfp4_quantize_act_desc q {};
    q.x = d->hidden;
    q.packed = d->hidden_packed;
    q.scale_linear = d->hidden_scale;
    q.global_scale = d->act_global_scale;
    q.rows = d->num_tokens;
    cudaStream_t main_stream = ctx->stream;
    const bool fork = quantise && !stage_recording() && plan_side_stream(plan);
    if (fork) {
        cudaError_t ferr = cudaEventRecord(plan->ev_fork, main_stream);
        if (ferr == cudaSuccess)
            ferr = cudaStreamWaitEvent(plan->side_stream, plan->ev_fork, 0);
        if (ferr != cudaSuccess)
            return set_cuda_error(ctx, ferr, "MoE route fork");
        ctx->stream = plan->side_stream;
        status = qs3_nvfp4_quantize_act(ctx, &q);
        ctx->stream = main_stream;
        if (status != QSFI_STATUS_OK)
            return status;
        ferr = cudaEventRecord(plan->ev_quant, plan->side_stream);
        if (ferr != cudaSuccess)
            return set_cuda_error(ctx, ferr, "MoE route fork");
    }

    GemmProblem gl {};
    gl.a = d->hidden.data;
    gl.a_rows = d->num_tokens;
    gl.a_pitch_bytes = static_cast<uint64_t>(h) * 2;
    gl.b = d->router_weight.data;
    gl.b_pitch_bytes = static_cast<uint64_t>(h) * 2;
    gl.groups = 1;
    gl.n = num_router_experts;
    gl.k = p.hidden_size;
    gl.epilogue = EPI_STORE_F32;
    gl.out = d->router_logits.data;
    gl.out_pitch_elems = num_router_experts;
    status = gemm_or_error(ctx, gl, "MoE router-logits GEMM");
    if (status != QSFI_STATUS_OK)
        return status;
    cudaError_t err = launch_router_topk(d->router_logits.data, 0, static_cast<const float*>(d->router_bias.data),
                                         static_cast<int32_t*>(d->topk_ids.data),
                                         static_cast<float*>(d->topk_weights.data), d->num_tokens,
                                         num_router_experts, p.top_k, d->score == QSCU_ROUTER_SCORE_SIGMOID,
                                         d->renormalize != 0, d->routed_scaling_factor, ctx->stream);
    if (err == cudaSuccess && (mapped || d->rank_mask.data != nullptr))
        err = launch_ep_route_targets(static_cast<const int32_t*>(d->topk_ids.data),
                                      static_cast<const int32_t*>(d->expert_id_map.data), num_router_experts,
                                      static_cast<int32_t*>(d->dispatch_ids.data),
                                      static_cast<uint32_t*>(d->rank_mask.data), d->num_tokens, p.top_k,
                                      p.local_num_experts, d->num_ranks, ctx->stream);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "MoE routing");
    if (fork)
        return set_cuda_error(ctx, cudaStreamWaitEvent(main_stream, plan->ev_quant, 0), "MoE route join");
    if (quantise)
        return qs3_nvfp4_quantize_act(ctx, &q);
    return QSFI_STATUS_OK;
}

qsfi_status qs3_moe_execute_nvfp4_prepared(qsfi_context* ctx, const qsfi_moe_plan* plan,
                                           const qs3_moe_nvfp4_prepared_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (plan == nullptr || d == nullptr)
        return set_invalid_arg(ctx, "plan/desc is null");
    const qsfi_moe_plan_desc& p = plan->desc;
    if (p.backend != QSFI_MOE_BACKEND_FLASHINFER_NVFP4)
        return set_invalid_arg(ctx, "qs3_moe_execute_nvfp4_prepared requires an NVFP4 MoE plan");
    if (d->num_tokens == 0 || d->num_tokens > p.max_num_tokens)
        return set_invalid_arg(ctx, "invalid MoE num_tokens");
    const int64_t t = d->num_tokens, h = p.hidden_size, i = p.intermediate_size, e = p.local_num_experts;
    status = validate_tensor(ctx, d->hidden_packed, "hidden_packed", QSFI_DTYPE_U8);
    if (status == QSFI_STATUS_OK)
        status = validate_tensor(ctx, d->hidden_scale, "hidden_scale", QSFI_DTYPE_FP8_E4M3);
    if (status == QSFI_STATUS_OK)
        status = validate_tensor(ctx, d->gate_up_weight, "gate_up_weight", QSFI_DTYPE_U8);
    if (status == QSFI_STATUS_OK)
        status = validate_tensor(ctx, d->down_weight, "down_weight", QSFI_DTYPE_U8);
    if (status == QSFI_STATUS_OK)
        status = validate_routing_tensors(ctx, p, d->num_tokens, d->topk_ids, d->topk_weights, d->out);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!contiguous2(d->hidden_packed) || !contiguous2(d->hidden_scale) || !contiguous3(d->gate_up_weight)
        || !contiguous3(d->down_weight))
        return set_invalid_arg(ctx, "NVFP4 MoE tensors must be contiguous");
    if (d->hidden_packed.shape[0] != t || d->hidden_packed.shape[1] != h / 2 || d->hidden_scale.shape[0] != t
        || d->hidden_scale.shape[1] != h / 16)
        return set_invalid_arg(ctx, "NVFP4 MoE hidden tensor shape mismatch");
    if (d->gate_up_weight.shape[0] != e || d->gate_up_weight.shape[1] != 2 * i
        || d->gate_up_weight.shape[2] != h / 2 || d->down_weight.shape[0] != e || d->down_weight.shape[1] != h
        || d->down_weight.shape[2] != i / 2)
        return set_invalid_arg(ctx, "NVFP4 MoE expert weight shape mismatch");
    status = validate_nvfp4_dims(ctx, p.hidden_size, p.intermediate_size, "");
    if (status != QSFI_STATUS_OK)
        return status;
    if (d->gate_up_scale_tiled.data == nullptr || d->down_scale_tiled.data == nullptr
        || static_cast<uint64_t>(d->gate_up_scale_tiled.shape[0]) < e * qs3_nvfp4_tiled_scale_bytes(2 * i, h)
        || static_cast<uint64_t>(d->down_scale_tiled.shape[0]) < e * qs3_nvfp4_tiled_scale_bytes(h, i))
        return set_invalid_arg(ctx, "NVFP4 MoE needs tiled weight scales of the right size");
    if (!gate_up_global_ok(d->gate_up_global_scale, e)
        || (d->down_global_scale.data != nullptr
            && (d->down_global_scale.dtype != QSFI_DTYPE_F32 || d->down_global_scale.shape[0] != e
                || !contiguous1(d->down_global_scale))))
        return set_invalid_arg(ctx, "global scales must be contiguous f32 [local_num_experts] tensors "
                                    "(gate_up: or [2 * local_num_experts])");
    const size_t need = carve_nvfp4(nullptr, p, d->num_tokens, false).bytes;
    status = validate_workspace(ctx, d->workspace, need);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_limits(ctx, p, d->num_tokens);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!aligned16(d->hidden_packed.data) || !aligned16(d->out.data) || !aligned16(d->gate_up_weight.data)
        || !aligned16(d->down_weight.data) || (reinterpret_cast<uintptr_t>(d->hidden_scale.data) & 3u) != 0)
        return set_invalid_arg(ctx, "NVFP4 MoE tensors must be 16-byte aligned (scales 4-byte aligned)");

    Nvfp4Workspace w = carve_nvfp4(static_cast<char*>(d->workspace.data), p, d->num_tokens, false);
    const uint32_t routes = d->num_tokens * p.top_k;
    cudaStream_t st = ctx->stream;
    stage_mark(st, STAGE_ROUTE_SORT);
    cudaError_t err = launch_route_sort(static_cast<const int32_t*>(d->topk_ids.data),
                                        static_cast<const float*>(d->topk_weights.data), routes, p.top_k,
                                        p.local_expert_offset, p.local_num_experts, w.rt, st);
    stage_mark(st, STAGE_GATHER);
    if (err == cudaSuccess)
        err = launch_nvfp4_gather_tiles(static_cast<const uint8_t*>(d->hidden_packed.data),
                                        static_cast<const uint8_t*>(d->hidden_scale.data), w.rt, routes,
                                        p.top_k, p.hidden_size, w.xq, w.xq_sf, st);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "NVFP4 MoE routing");
    Nvfp4Weights wt {};
    wt.gu_packed = static_cast<const uint8_t*>(d->gate_up_weight.data);
    wt.gu_sf_tiled = static_cast<const uint8_t*>(d->gate_up_scale_tiled.data);
    wt.gu_global = static_cast<const float*>(d->gate_up_global_scale.data);
    wt.gu_global_up = gate_up_global_up(d->gate_up_global_scale, p.local_num_experts);
    wt.d_packed = static_cast<const uint8_t*>(d->down_weight.data);
    wt.d_sf_tiled = static_cast<const uint8_t*>(d->down_scale_tiled.data);
    wt.d_global = static_cast<const float*>(d->down_global_scale.data);
    status = run_routed_nvfp4(ctx, p, w, wt, d->act_global_scale, d->act2_global_scale);
    if (status != QSFI_STATUS_OK)
        return status;
    CombineParams cp {};
    cp.route_prows = w.rt.route_prows;
    cp.topk_weights = static_cast<const float*>(d->topk_weights.data);
    cp.expert_out = w.y2;
    cp.out = static_cast<__nv_bfloat16*>(d->out.data);
    cp.num_tokens = d->num_tokens;
    cp.top_k = p.top_k;
    cp.hidden_size = p.hidden_size;
    cp.skip_empty = (d->flags & 1u) != 0;
    stage_mark(st, STAGE_COMBINE);
    err = launch_combine(cp, st);
    stage_mark(st, STAGE_END);
    return set_cuda_error(ctx, err, "qs3_moe_execute_nvfp4_prepared");
}

qsfi_status qs3_moe_ep_finish_workspace_size(qsfi_context* ctx, const qsfi_moe_plan* plan, uint32_t num_tokens,
                                             uint32_t num_ranks, uint32_t shared_intermediate_size,
                                             size_t* device_bytes)
{
    if (device_bytes == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    *device_bytes = 0;
    if (ctx == nullptr || plan == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    if (num_tokens == 0 || num_ranks == 0 || num_ranks > 32)
        return set_invalid_arg(ctx, "invalid expert-parallel finish dimensions");
    const size_t routes = static_cast<size_t>(num_tokens) * num_ranks;
    size_t off = 0;
    carve<int32_t>(nullptr, off, routes);
    carve<float>(nullptr, off, routes);
    const size_t base = align_up(off, kWorkspaceAlign);
    *device_bytes = carve_layer(nullptr, base, plan->desc, num_tokens, shared_intermediate_size, true).bytes;
    return QSFI_STATUS_OK;
}

qsfi_status qs3_moe_ep_finish(qsfi_context* ctx, const qsfi_moe_plan* plan, const qs3_moe_ep_finish_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (plan == nullptr || d == nullptr)
        return set_invalid_arg(ctx, "plan/desc is null");
    const qsfi_moe_plan_desc& p = plan->desc;
    if (p.backend != QSFI_MOE_BACKEND_FLASHINFER_NVFP4)
        return set_invalid_arg(ctx, "qs3_moe_ep_finish requires an NVFP4 MoE plan");
    if (d->num_tokens == 0 || d->num_ranks == 0 || d->num_ranks > 32 || (d->phases & 3u) == 0)
        return set_invalid_arg(ctx, "invalid expert-parallel finish dimensions");
    const int64_t t = d->num_tokens, h = p.hidden_size;
    const uint32_t is = d->shared_intermediate_size;
    const bool shared = d->shared_gate_up_weight.data != nullptr;
    status = validate_tensor(ctx, d->hidden, "hidden", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!contiguous2(d->hidden) || d->hidden.shape[0] != t || d->hidden.shape[1] != h)
        return set_invalid_arg(ctx, "MoE token/top-k tensor shape mismatch");
    if (shared) {
        if (is == 0 || is % 256 != 0)
            return set_invalid_arg(ctx, "invalid shared_intermediate_size");
        status = validate_tensor(ctx, d->shared_gate_up_weight, "shared_gate_up_weight", QSFI_DTYPE_U8);
        if (status == QSFI_STATUS_OK)
            status = validate_tensor(ctx, d->shared_down_weight, "shared_down_weight", QSFI_DTYPE_U8);
        if (status == QSFI_STATUS_OK)
            status = validate_tensor(ctx, d->shared_gate_weight, "shared_gate_weight", QSFI_DTYPE_BF16);
        if (status != QSFI_STATUS_OK)
            return status;
        if (!contiguous3(d->shared_gate_up_weight) || !contiguous3(d->shared_down_weight)
            || !contiguous2(d->shared_gate_weight) || d->shared_gate_up_weight.shape[0] != 1
            || d->shared_gate_up_weight.shape[1] != 2ll * is || d->shared_gate_up_weight.shape[2] != h / 2
            || d->shared_down_weight.shape[0] != 1 || d->shared_down_weight.shape[1] != h
            || d->shared_down_weight.shape[2] != is / 2 || d->shared_gate_weight.shape[0] != 1
            || d->shared_gate_weight.shape[1] != h)
            return set_invalid_arg(ctx, "MoE shared expert weight shape mismatch");
        if (d->shared_gate_up_scale_tiled.data == nullptr || d->shared_down_scale_tiled.data == nullptr
            || static_cast<uint64_t>(d->shared_gate_up_scale_tiled.shape[0]) < qs3_nvfp4_tiled_scale_bytes(2 * is, h)
            || static_cast<uint64_t>(d->shared_down_scale_tiled.shape[0]) < qs3_nvfp4_tiled_scale_bytes(h, is))
            return set_invalid_arg(ctx, "NVFP4 MoE layer needs tiled shared-expert scales of the right size");
        if (!gate_up_global_ok(d->shared_gate_up_global_scale, 1))
            return set_invalid_arg(ctx, "gate_up global scales must be contiguous f32 [groups] or [2 * groups] tensors");
        status = validate_nvfp4_dims(ctx, p.hidden_size, is, "shared-expert");
        if (status != QSFI_STATUS_OK)
            return status;
    }
    size_t need = 0;
    status = qs3_moe_ep_finish_workspace_size(ctx, plan, d->num_tokens, d->num_ranks, shared ? is : 0, &need);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_workspace(ctx, d->workspace, need);
    if (status != QSFI_STATUS_OK)
        return status;
    char* base = static_cast<char*>(d->workspace.data);
    size_t off = 0;
    const size_t routes = static_cast<size_t>(d->num_tokens) * d->num_ranks;
    int32_t* rows = carve<int32_t>(base, off, routes);
    float* ones = carve<float>(base, off, routes);
    LayerExtra x = carve_layer(base, align_up(off, kWorkspaceAlign), p, d->num_tokens, shared ? is : 0, true);
    cudaStream_t st = ctx->stream;
    const __nv_bfloat16* hidden = static_cast<const __nv_bfloat16*>(d->hidden.data);

    if ((d->phases & 1u) != 0 && shared) {
        cudaError_t err = launch_nvfp4_gather_quantize(hidden, nullptr, d->num_tokens, 1, p.hidden_size,
                                                       d->act_global_scale, x.sh_xq, x.sh_xq_sf, st);
        if (err != cudaSuccess)
            return set_cuda_error(ctx, err, "NVFP4 shared expert quantise");
        const float ga = d->act_global_scale == 0.0f ? 1.0f : d->act_global_scale;
        const float ga2 = d->act2_global_scale == 0.0f ? 1.0f : d->act2_global_scale;
        GemmProblem s1 {};
        s1.nvfp4 = 1;
        s1.a = x.sh_xq;
        s1.a_rows = d->num_tokens;
        s1.a_pitch_bytes = h / 2;
        s1.a_scale_tiled = x.sh_xq_sf;
        s1.b = d->shared_gate_up_weight.data;
        s1.b_pitch_bytes = h / 2;
        s1.b_scale_tiled = static_cast<const uint8_t*>(d->shared_gate_up_scale_tiled.data);
        s1.groups = 1;
        s1.n = is;
        s1.k = p.hidden_size;
        s1.gated = 1;
        s1.epilogue = EPI_SWIGLU_NVFP4;
        s1.out = x.sh_actq;
        s1.out_pitch_elems = is / 2;
        s1.out_scale_tiled = x.sh_actq_sf;
        s1.alpha = ga;
        s1.group_scale = static_cast<const float*>(d->shared_gate_up_global_scale.data);
        s1.group_scale_up = gate_up_global_up(d->shared_gate_up_global_scale, 1);
        s1.out_global_scale = ga2;
        status = gemm_or_error(ctx, s1, "NVFP4 shared gate_up GEMM");
        if (status != QSFI_STATUS_OK)
            return status;
        GemmProblem s2 {};
        s2.nvfp4 = 1;
        s2.a = x.sh_actq;
        s2.a_rows = d->num_tokens;
        s2.a_pitch_bytes = is / 2;
        s2.a_scale_tiled = x.sh_actq_sf;
        s2.b = d->shared_down_weight.data;
        s2.b_pitch_bytes = is / 2;
        s2.b_scale_tiled = static_cast<const uint8_t*>(d->shared_down_scale_tiled.data);
        s2.groups = 1;
        s2.n = p.hidden_size;
        s2.k = is;
        s2.epilogue = EPI_STORE_BF16;
        s2.out = x.sh_out;
        s2.out_pitch_elems = p.hidden_size;
        s2.alpha = ga2;
        s2.group_scale = static_cast<const float*>(d->shared_down_global_scale.data);
        status = gemm_or_error(ctx, s2, "NVFP4 shared down GEMM");
        if (status != QSFI_STATUS_OK)
            return status;
    }
    if ((d->phases & 2u) != 0 && d->peer_partials != nullptr) {
        // pull mode: read the ranks' partial sums in place through peer-mapped pointers
        status = validate_tensor(ctx, d->out, "out", QSFI_DTYPE_BF16);
        if (status == QSFI_STATUS_OK)
            status = validate_tensor(ctx, d->topk_ids, "topk_ids", QSFI_DTYPE_I32);
        if (status != QSFI_STATUS_OK)
            return status;
        if (!contiguous2(d->out) || d->out.shape[0] != t || d->out.shape[1] != h || !contiguous2(d->topk_ids)
            || d->topk_ids.shape[0] != t || d->topk_ids.shape[1] != p.top_k)
            return set_invalid_arg(ctx, "MoE token/top-k tensor shape mismatch");
        if (static_cast<uint64_t>(p.local_num_experts) * d->num_ranks != p.num_experts
            || p.local_expert_offset % p.local_num_experts != 0)
            return set_invalid_arg(ctx, "pull combine needs equal contiguous expert blocks per rank");
        EpPullParams pp {};
        for (uint32_t r = 0; r < d->num_ranks; ++r) {
            if (d->peer_partials[r] == nullptr || !aligned16(d->peer_partials[r]))
                return set_invalid_arg(ctx, "peer_partials entries must be 16-byte aligned device pointers");
            pp.peer[r] = static_cast<const __nv_bfloat16*>(d->peer_partials[r]);
        }
        pp.topk_ids = static_cast<const int32_t*>(d->topk_ids.data);
        pp.out = static_cast<__nv_bfloat16*>(d->out.data);
        if (shared) {
            pp.shared_out = x.sh_out;
            pp.hidden = hidden;
            pp.gate_w = static_cast<const __nv_bfloat16*>(d->shared_gate_weight.data);
        }
        pp.num_tokens = d->num_tokens;
        pp.top_k = p.top_k;
        pp.hidden_size = p.hidden_size;
        pp.num_ranks = d->num_ranks;
        pp.my_rank = p.local_expert_offset / p.local_num_experts;
        pp.experts_per_rank = p.local_num_experts;
        return set_cuda_error(ctx, launch_ep_pull_combine(pp, st), "qs3_moe_ep_finish");
    }
    if ((d->phases & 2u) != 0) {
        status = validate_tensor(ctx, d->partials, "partials", QSFI_DTYPE_BF16);
        if (status == QSFI_STATUS_OK)
            status = validate_tensor(ctx, d->out, "out", QSFI_DTYPE_BF16);
        if (status != QSFI_STATUS_OK)
            return status;
        if (!contiguous3(d->partials) || d->partials.shape[0] != d->num_ranks || d->partials.shape[1] != t
            || d->partials.shape[2] != h || !contiguous2(d->out) || d->out.shape[0] != t || d->out.shape[1] != h)
            return set_invalid_arg(ctx, "expert-parallel partial-sum tensor shape mismatch");
        if (!aligned16(d->partials.data) || !aligned16(d->out.data))
            return set_invalid_arg(ctx, "MoE tensors must be 16-byte aligned");
        // out[t] = sum over source ranks r (ascending) of partials[r][t]: the combine
        // kernel with one unit-weight "route" per rank pointing at row r * T + t
        cudaError_t err = launch_ep_rank_routes(rows, ones, d->num_tokens, d->num_ranks, st);
        if (err != cudaSuccess)
            return set_cuda_error(ctx, err, "expert-parallel combine setup");
        CombineParams cp {};
        cp.route_prows = rows;
        cp.topk_weights = ones;
        cp.expert_out = static_cast<const __nv_bfloat16*>(d->partials.data);
        cp.out = static_cast<__nv_bfloat16*>(d->out.data);
        cp.num_tokens = d->num_tokens;
        cp.top_k = d->num_ranks;
        cp.hidden_size = p.hidden_size;
        if (shared) {
            cp.shared_out = x.sh_out;
            cp.hidden = hidden;
            cp.gate_w = static_cast<const __nv_bfloat16*>(d->shared_gate_weight.data);
        }
        return set_cuda_error(ctx, launch_combine(cp, st), "qs3_moe_ep_finish");
    }
    return QSFI_STATUS_OK;
}

qsfi_status qs3_moe_ep_pull_tokens(qsfi_context* ctx, const qs3_moe_ep_pull_tokens_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d == nullptr || d->peer_blocks == nullptr)
        return set_invalid_arg(ctx, "desc/peer_blocks is null");
    if (d->num_ranks == 0 || d->num_ranks > 32 || d->num_segments == 0 || d->num_segments > 4)
        return set_invalid_arg(ctx, "expert-parallel pull: 1..32 ranks and 1..4 segments");
    EpPullTokensParams p {};
    p.num_ranks = d->num_ranks;
    p.num_segments = d->num_segments;
    for (uint32_t r = 0; r < d->num_ranks; ++r) {
        if (d->peer_blocks[r] == nullptr || !aligned16(d->peer_blocks[r]))
            return set_invalid_arg(ctx, "expert-parallel pull: peer blocks must be non-null and 16-byte aligned");
        p.peer[r] = static_cast<const uint8_t*>(d->peer_blocks[r]);
    }
    for (uint32_t j = 0; j < d->num_segments; ++j) {
        if (d->dst[j] == nullptr || !aligned16(d->dst[j]) || d->segment_offset[j] % 16 != 0
            || d->segment_bytes[j] % 16 != 0)
            return set_invalid_arg(ctx, "expert-parallel pull: segments must be 16-byte aligned and sized");
        p.seg_offset[j] = d->segment_offset[j];
        p.seg_bytes[j] = d->segment_bytes[j];
        p.dst[j] = static_cast<uint8_t*>(d->dst[j]);
    }
    return set_cuda_error(ctx, launch_ep_pull_tokens(p, ctx->stream), "qs3_moe_ep_pull_tokens");
}

qsfi_status qs3_moe_ep_pull_routed(qsfi_context* ctx, const qs3_moe_ep_pull_routed_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d == nullptr || d->peer_blocks == nullptr)
        return set_invalid_arg(ctx, "desc/peer_blocks is null");
    if (d->num_ranks == 0 || d->num_ranks > 32 || d->my_rank >= d->num_ranks || d->num_tokens == 0 || d->top_k == 0
        || d->top_k > 16 || d->hidden_size == 0 || d->hidden_size % 256 != 0 || d->hidden_size > 2048)
        return set_invalid_arg(ctx, "expert-parallel pull: 1..32 ranks, top_k <= 16, hidden a multiple of 256 up to 2048");
    if (static_cast<uint64_t>(d->num_ranks) * d->num_tokens > 0x7fffffffull / 16)
        return set_unsupported(ctx, "expert-parallel pull: too many token rows");
    EpPullRoutedParams p {};
    for (uint32_t r = 0; r < d->num_ranks; ++r) {
        if (d->peer_blocks[r] == nullptr || !aligned16(d->peer_blocks[r]))
            return set_invalid_arg(ctx, "expert-parallel pull: peer blocks must be non-null and 16-byte aligned");
        p.peer[r] = static_cast<const uint8_t*>(d->peer_blocks[r]);
    }
    if ((d->offset_codes | d->offset_scales | d->offset_ids | d->offset_weights | d->offset_mask) % 16 != 0
        || !aligned16(d->dst_codes) || !aligned16(d->dst_scales) || !aligned16(d->dst_ids) || !aligned16(d->dst_weights)
        || d->dst_codes == nullptr || d->dst_scales == nullptr || d->dst_ids == nullptr || d->dst_weights == nullptr)
        return set_invalid_arg(ctx, "expert-parallel pull: segments and destinations must be 16-byte aligned");
    p.off_codes = d->offset_codes;
    p.off_scales = d->offset_scales;
    p.off_ids = d->offset_ids;
    p.off_wts = d->offset_weights;
    p.off_mask = d->offset_mask;
    p.dst_codes = static_cast<uint8_t*>(d->dst_codes);
    p.dst_scales = static_cast<uint8_t*>(d->dst_scales);
    p.dst_ids = static_cast<uint8_t*>(d->dst_ids);
    p.dst_wts = static_cast<uint8_t*>(d->dst_weights);
    p.num_ranks = d->num_ranks;
    p.my_rank = d->my_rank;
    p.num_tokens = d->num_tokens;
    p.top_k = d->top_k;
    p.code_vecs = d->hidden_size / 32;
    p.scale_vecs = d->hidden_size / 256;
    return set_cuda_error(ctx, launch_ep_pull_routed(p, ctx->stream), "qs3_moe_ep_pull_routed");
}

// ---- FP8 block-scaled path ------------------------------------------------------------

qsfi_status qs3_fp8_quantize_weight(qsfi_context* ctx, const qs3_fp8_quantize_weight_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d == nullptr)
        return set_invalid_arg(ctx, "desc is null");
    status = validate_tensor(ctx, d->weight, "weight", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, d->codes, "codes", QSFI_DTYPE_FP8_E4M3);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, d->scale, "scale", QSFI_DTYPE_F32);
    if (status != QSFI_STATUS_OK)
        return status;
    const int64_t e = d->weight.shape[0], rows = d->weight.shape[1], k = d->weight.shape[2];
    if (!contiguous3(d->weight) || !contiguous3(d->codes) || !contiguous3(d->scale))
        return set_invalid_arg(ctx, "FP8 weight quantiser tensors must be contiguous");
    if (k % 128 != 0 || e > 65535 || (rows + 127) / 128 > 65535)
        return set_invalid_arg(ctx, "FP8 weight quantiser needs k divisible by 128");
    if (d->codes.shape[0] != e || d->codes.shape[1] != rows || d->codes.shape[2] != k || d->scale.shape[0] != e
        || d->scale.shape[1] != (rows + 127) / 128 || d->scale.shape[2] != k / 128)
        return set_invalid_arg(ctx, "FP8 weight quantiser tensor shape mismatch");
    if (!aligned16(d->weight.data) || !aligned16(d->codes.data))
        return set_invalid_arg(ctx, "FP8 weight quantiser tensors must be 16-byte aligned");
    return set_cuda_error(ctx,
                          launch_fp8_quantize_weight(static_cast<const __nv_bfloat16*>(d->weight.data),
                                                     static_cast<uint32_t>(e), static_cast<uint32_t>(rows),
                                                     static_cast<uint32_t>(k), static_cast<uint8_t*>(d->codes.data),
                                                     static_cast<float*>(d->scale.data), ctx->stream),
                          "qs3_fp8_quantize_weight");
}

qsfi_status qs3_fp8_quantize_act(qsfi_context* ctx, const qs3_fp8_quantize_act_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d == nullptr)
        return set_invalid_arg(ctx, "desc is null");
    status = validate_tensor(ctx, d->x, "x", QSFI_DTYPE_BF16);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, d->codes, "codes", QSFI_DTYPE_FP8_E4M3);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, d->scale, "scale", QSFI_DTYPE_F32);
    if (status != QSFI_STATUS_OK)
        return status;
    const int64_t rows = d->rows, k = d->x.shape[1];
    if (!contiguous2(d->x) || !contiguous2(d->codes) || !contiguous2(d->scale))
        return set_invalid_arg(ctx, "FP8 activation quantiser tensors must be contiguous");
    if (rows == 0 || k % 128 != 0 || d->x.shape[0] < rows || d->codes.shape[0] < rows || d->codes.shape[1] != k
        || d->scale.shape[0] < rows || d->scale.shape[1] != k / 128)
        return set_invalid_arg(ctx, "FP8 activation quantiser tensor shape mismatch");
    if ((reinterpret_cast<uintptr_t>(d->x.data) & 7u) != 0 || (reinterpret_cast<uintptr_t>(d->codes.data) & 3u) != 0)
        return set_invalid_arg(ctx, "FP8 activation quantiser tensors must be 8-byte aligned");
    return set_cuda_error(ctx,
                          launch_fp8_gather_quantize(static_cast<const __nv_bfloat16*>(d->x.data), nullptr,
                                                     static_cast<uint32_t>(rows), 1, static_cast<uint32_t>(k),
                                                     static_cast<uint8_t*>(d->codes.data),
                                                     static_cast<float*>(d->scale.data), ctx->stream),
                          "qs3_fp8_quantize_act");
}

qsfi_status qs3_moe_execute_fp8(qsfi_context* ctx, const qsfi_moe_plan* plan, const qs3_moe_fp8_execute_desc* desc)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    if (plan == nullptr || desc == nullptr)
        return set_invalid_arg(ctx, "plan/desc is null");
    const qsfi_moe_plan_desc& p = plan->desc;
    if (!is_fp8_plan(p))
        return set_invalid_arg(ctx, "qs3_moe_execute_fp8 requires an FP8 block-scaled MoE plan");
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (desc->num_tokens == 0 || desc->num_tokens > p.max_num_tokens)
        return set_invalid_arg(ctx, "invalid MoE num_tokens");
    const int64_t t = desc->num_tokens, h = p.hidden_size, i = p.intermediate_size, e = p.local_num_experts;
    status = validate_tensor(ctx, desc->hidden, "hidden", QSFI_DTYPE_FP8_E4M3);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->hidden_scale, "hidden_scale", QSFI_DTYPE_F32);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->gate_up_weight, "gate_up_weight", QSFI_DTYPE_FP8_E4M3);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->gate_up_weight_scale, "gate_up_weight_scale", QSFI_DTYPE_F32);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->down_weight, "down_weight", QSFI_DTYPE_FP8_E4M3);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_tensor(ctx, desc->down_weight_scale, "down_weight_scale", QSFI_DTYPE_F32);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_routing_tensors(ctx, p, desc->num_tokens, desc->topk_ids, desc->topk_weights, desc->out);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!contiguous2(desc->hidden) || !contiguous2(desc->hidden_scale) || !contiguous3(desc->gate_up_weight)
        || !contiguous3(desc->gate_up_weight_scale) || !contiguous3(desc->down_weight)
        || !contiguous3(desc->down_weight_scale))
        return set_invalid_arg(ctx, "FP8 MoE tensors must be contiguous");
    if (desc->hidden.shape[0] != t || desc->hidden.shape[1] != h || desc->hidden_scale.shape[0] != t
        || desc->hidden_scale.shape[1] != h / 128)
        return set_invalid_arg(ctx, "FP8 MoE hidden tensor shape mismatch");
    if (desc->gate_up_weight.shape[0] != e || desc->gate_up_weight.shape[1] != 2 * i
        || desc->gate_up_weight.shape[2] != h || desc->gate_up_weight_scale.shape[0] != e
        || desc->gate_up_weight_scale.shape[1] != 2 * i / 128 || desc->gate_up_weight_scale.shape[2] != h / 128
        || desc->down_weight.shape[0] != e || desc->down_weight.shape[1] != h || desc->down_weight.shape[2] != i
        || desc->down_weight_scale.shape[0] != e || desc->down_weight_scale.shape[1] != h / 128
        || desc->down_weight_scale.shape[2] != i / 128)
        return set_invalid_arg(ctx, "FP8 MoE expert weight shape mismatch");
    size_t need = 0;
    status = qsfi_moe_workspace_size(ctx, plan, desc->num_tokens, &need);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_workspace(ctx, desc->workspace, need);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_limits(ctx, p, desc->num_tokens);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!aligned16(desc->hidden.data) || !aligned16(desc->out.data) || !aligned16(desc->gate_up_weight.data)
        || !aligned16(desc->down_weight.data))
        return set_invalid_arg(ctx, "FP8 MoE tensors must be 16-byte aligned");

    status = validate_routes_checked(ctx, p, desc->topk_ids.data, desc->topk_weights.data,
                                     desc->num_tokens * p.top_k);
    if (status != QSFI_STATUS_OK)
        return status;
    Fp8Workspace w = carve_fp8(static_cast<char*>(desc->workspace.data), p, desc->num_tokens);
    const uint32_t routes = desc->num_tokens * p.top_k;
    cudaStream_t st = ctx->stream;
    cudaError_t err = launch_route_sort(static_cast<const int32_t*>(desc->topk_ids.data),
                                        static_cast<const float*>(desc->topk_weights.data), routes, p.top_k,
                                        p.local_expert_offset, p.local_num_experts, w.rt, st);
    // gather the quantised token rows (codes and their scales) into expert order
    if (err == cudaSuccess)
        err = launch_gather_rows(desc->hidden.data, static_cast<uint32_t>(h), w.rt.route_prows, routes, p.top_k,
                                 w.xq, st);
    if (err == cudaSuccess)
        err = launch_gather_rows(desc->hidden_scale.data, static_cast<uint32_t>(h / 128 * 4), w.rt.route_prows,
                                 routes, p.top_k, w.xq_s, st);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "FP8 MoE routing");
    status = run_routed_fp8(ctx, p, w, desc->num_tokens, static_cast<const uint8_t*>(desc->gate_up_weight.data),
                            static_cast<const float*>(desc->gate_up_weight_scale.data),
                            static_cast<const uint8_t*>(desc->down_weight.data),
                            static_cast<const float*>(desc->down_weight_scale.data));
    if (status != QSFI_STATUS_OK)
        return status;
    CombineParams cp {};
    cp.route_prows = w.rt.route_prows;
    cp.topk_weights = static_cast<const float*>(desc->topk_weights.data);
    cp.expert_out = w.y2;
    cp.out = static_cast<__nv_bfloat16*>(desc->out.data);
    cp.num_tokens = desc->num_tokens;
    cp.top_k = p.top_k;
    cp.hidden_size = p.hidden_size;
    return set_cuda_error(ctx, launch_combine(cp, st), "qs3_moe_execute_fp8");
}

// earlier name of the same entry point
qsfi_status qsfi_moe_execute_fp8(qsfi_context* ctx, const qsfi_moe_plan* plan, const qsfi_moe_fp8_execute_desc* desc)
{
    return qs3_moe_execute_fp8(ctx, plan, desc);
}

} // extern "C"
