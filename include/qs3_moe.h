/*
 * qs3_moe.h -- C ABI of the sm_100a mixture-of-experts library (libqs3moe.so).
 *
 * Two groups of declarations live here:
 *
 *  1. The part of the qs3 ("quasar3") kernel boundary that its MoE layer goes
 *     through. Struct layouts, enum values, symbol names and error behaviour
 *     follow the upstream headers so that objects built from this library can
 *     replace the upstream MoE/router objects at link time. Every such
 *     declaration cites the upstream file:line it is layout-compatible with.
 *
 *  2. Additive entry points (prefix qs3_) that upstream does not have: NVFP4
 *     weight preparation, a dense bf16 GEMM for the router / shared expert, a
 *     whole-layer call (router logits -> top-k -> experts -> combine), the
 *     expert-parallel pack/unpack helpers, and a checkpoint loader for the
 *     tensors of one MoE layer. They never change an upstream signature.
 *
 * Conventions (upstream qs_tensor.h:6-13, qsfi.h:14-18): strides are element
 * strides; an optional tensor is absent when data == NULL; all work is
 * enqueued on the stream owned by the context (or passed explicitly for the
 * context-free qscu_ helpers) and nothing synchronises in release builds.
 */
#ifndef QS3_MOE_H
#define QS3_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- status -- */

#define QSFI_ERROR_MESSAGE_BYTES 512u /* upstream qs_info.h:10 */

/* Checked builds add device-side validation plus one stream sync per validated
 * call (upstream qs_info.h:12-18). The shipped library is a release build. */
#ifndef QSFI_ENABLE_CHECKED_VALIDATION
#define QSFI_ENABLE_CHECKED_VALIDATION 0
#endif

typedef enum { /* upstream qs_info.h:20-28 */
    QSFI_STATUS_OK = 0,
    QSFI_STATUS_INVALID_ARGUMENT = 1,
    QSFI_STATUS_UNSUPPORTED = 2,
    QSFI_STATUS_OUT_OF_MEMORY = 3,
    QSFI_STATUS_CUDA_ERROR = 4,
    QSFI_STATUS_BACKEND_ERROR = 5,
    QSFI_STATUS_INTERNAL_ERROR = 6
} qsfi_status;

typedef enum { /* upstream qs_info.h:30-36 */
    QSFI_ERROR_SOURCE_NONE = 0,
    QSFI_ERROR_SOURCE_QSFI = 1,
    QSFI_ERROR_SOURCE_CUDA = 2,
    QSFI_ERROR_SOURCE_FLASHINFER = 3,
    QSFI_ERROR_SOURCE_CUBLASLT = 4
} qsfi_error_source;

typedef struct { /* upstream qs_info.h:38-43 */
    qsfi_status status;
    qsfi_error_source source;
    int32_t native_code;
    char message[QSFI_ERROR_MESSAGE_BYTES];
} qsfi_error_info;

const char* qsfi_status_string(qsfi_status status); /* upstream qs_info.h:45 */

/* --------------------------------------------------------------- tensors -- */

typedef void* qsfi_cuda_stream; /* upstream qs_tensor.h:12 */
typedef void* qsfi_device_ptr;  /* upstream qs_tensor.h:13 */

typedef enum { /* upstream qs_tensor.h:15-29 */
    QSFI_DTYPE_INVALID = 0,
    QSFI_DTYPE_F32 = 1,
    QSFI_DTYPE_F16 = 2,
    QSFI_DTYPE_BF16 = 3,
    QSFI_DTYPE_FP8_E4M3 = 4,
    QSFI_DTYPE_FP8_E5M2 = 5,
    QSFI_DTYPE_NVFP4_E2M1 = 6,
    QSFI_DTYPE_MXFP4_E2M1 = 7,
    QSFI_DTYPE_MXFP8_E4M3 = 8,
    QSFI_DTYPE_I32 = 9,
    QSFI_DTYPE_U32 = 10,
    QSFI_DTYPE_I8 = 11,
    QSFI_DTYPE_U8 = 12
} qsfi_dtype;

/* Rank-N strided views, upstream qs_tensor.h:31-50. */
#define QS3_DECLARE_TENSOR(N)                                                                      \
    typedef struct {                                                                               \
        qsfi_device_ptr data;                                                                      \
        qsfi_dtype dtype;                                                                          \
        int64_t shape[N];                                                                          \
        int64_t stride[N];                                                                         \
    } qsfi_tensor##N
QS3_DECLARE_TENSOR(1);
QS3_DECLARE_TENSOR(2);
QS3_DECLARE_TENSOR(3);
#undef QS3_DECLARE_TENSOR

/* --------------------------------------------------------------- context -- */

typedef struct qsfi_context qsfi_context;   /* upstream qsfi.h:20 */
typedef struct qsfi_moe_plan qsfi_moe_plan; /* upstream qsfi.h:23 */

typedef struct { /* upstream qsfi.h:33-36 */
    int32_t device_ordinal; /* < 0: whatever device is current at call time. */
    qsfi_cuda_stream stream; /* NULL: the default stream. */
} qsfi_context_desc;

typedef struct { /* upstream qsfi.h:38-46 */
    uint32_t target_sm;
    uint32_t target_compute_capability_major;
    uint32_t target_compute_capability_minor;
    uint32_t assume_fp8;
    uint32_t assume_fp4;
    uint32_t assume_pdl;
    uint32_t gemm_backend;
} qsfi_build_config;

typedef struct { /* upstream qsfi.h:48-51 */
    uint32_t runtime_compute_capability_major;
    uint32_t runtime_compute_capability_minor;
} qsfi_context_info;

/* Context life cycle and error read-back, upstream qsfi.h:268-288 and
 * qsfi_context.cu:120-283. This build answers target_sm = 100 (CC 10.0). */
qsfi_status qsfi_context_create(const qsfi_context_desc* desc, qsfi_context** out);
void qsfi_context_destroy(qsfi_context* ctx);
qsfi_status qsfi_context_set_stream(qsfi_context* ctx, qsfi_cuda_stream stream);
qsfi_status qsfi_get_build_config(qsfi_build_config* out);
qsfi_status qsfi_context_get_info(qsfi_context* ctx, qsfi_context_info* out);
qsfi_status qsfi_context_validate_target(qsfi_context* ctx);
qsfi_status qsfi_context_get_last_error(const qsfi_context* ctx, qsfi_error_info* out);
void qsfi_context_clear_last_error(qsfi_context* ctx);

/* ------------------------------------------------------------ MoE (qsfi) -- */

typedef enum { /* upstream qsfi.h:211-215; the names keep upstream's spelling */
    QSFI_MOE_BACKEND_FLASHINFER_STAGED_BF16 = 1,
    QSFI_MOE_BACKEND_FLASHINFER_FUSED_BF16 = 2,
    QSFI_MOE_BACKEND_FLASHINFER_NVFP4 = 3
} qsfi_moe_backend;

typedef enum { /* upstream qsfi.h:217-220 */
    QSFI_MOE_ROUTE_PRECOMPUTED_TOPK = 0,
    QSFI_MOE_ROUTE_ROUTER_LOGITS = 1
} qsfi_moe_route_mode;

typedef struct { /* upstream qsfi.h:222-236 */
    qsfi_moe_backend backend;
    qsfi_moe_route_mode route_mode;
    uint32_t max_num_tokens;
    uint32_t hidden_size;
    uint32_t intermediate_size;
    uint32_t num_experts;
    uint32_t top_k;
    uint32_t local_expert_offset; /* first global expert id owned by this rank */
    uint32_t local_num_experts;
    qsfi_dtype activation_dtype;
    qsfi_dtype weight_dtype;
    qsfi_dtype output_dtype;
    uint32_t reserved0;
} qsfi_moe_plan_desc;

typedef struct { /* upstream qsfi.h:238-247 */
    qsfi_tensor2 hidden;         /* bf16 [num_tokens, hidden] */
    qsfi_tensor2 topk_ids;       /* i32  [num_tokens, top_k], GLOBAL expert ids */
    qsfi_tensor2 topk_weights;   /* f32  [num_tokens, top_k], final per-route scale */
    qsfi_tensor3 gate_up_weight; /* bf16 [local_experts, 2*inter, hidden]; rows [0,inter) gate */
    qsfi_tensor3 down_weight;    /* bf16 [local_experts, hidden, inter] */
    qsfi_tensor2 out;            /* bf16 [num_tokens, hidden] */
    qsfi_tensor1 workspace;      /* u8/i8 [>= qsfi_moe_workspace_size] */
    uint32_t num_tokens;
} qsfi_moe_bf16_execute_desc;

typedef struct { /* upstream qsfi.h:249-266 */
    qsfi_tensor2 hidden_packed;         /* u8   [num_tokens, hidden/2], low nibble = even k */
    qsfi_tensor2 hidden_scale;          /* e4m3 [num_tokens, hidden/16], row-major ("linear") */
    qsfi_tensor2 topk_ids;              /* i32  [num_tokens, top_k] */
    qsfi_tensor2 topk_weights;          /* f32  [num_tokens, top_k] */
    qsfi_tensor3 gate_up_weight_packed; /* u8   [local_experts, 2*inter, hidden/2] */
    qsfi_tensor3 gate_up_weight_scale;  /* e4m3 [local_experts, 2*inter, hidden/16], linear */
    qsfi_tensor3 down_weight_packed;    /* u8   [local_experts, hidden, inter/2] */
    qsfi_tensor3 down_weight_scale;     /* e4m3 [local_experts, hidden, inter/16], linear */
    qsfi_tensor1 expert_output_scale;   /* optional f32 [local_experts]: down-GEMM output scale */
    qsfi_tensor2 out;                   /* bf16 [num_tokens, hidden] */
    qsfi_tensor1 workspace;             /* u8/i8 */
    uint32_t num_tokens;
} qsfi_moe_nvfp4_execute_desc;

/* Plan and execute, upstream qsfi.h:333-344 (qsfi_moe.cu:730-821).
 *
 * Differences from upstream, all additive:
 *  - an expert-parallel plan (partial local expert range) is accepted: routes to
 *    non-local experts are skipped and `out` holds this rank's partial sum
 *    (upstream rejects such plans, qsfi_moe.cu:160-166, although its kernels
 *    already skip non-local routes, qsfi_moe.cu:340-343,379-381,484);
 *  - qsfi_moe_execute_nvfp4 is implemented (upstream returns UNSUPPORTED,
 *    qsfi_moe.cu:807-821) and qsfi_moe_workspace_size answers for NVFP4 plans;
 *  - the order of rows inside one expert's segment is deterministic (stable in
 *    route index); upstream's depends on atomics order (qsfi_moe.cu:378-382).
 * The reported BF16 workspace size is never smaller than upstream's formula
 * (qsfi_moe.cu:67-121), which the upstream Rust caller re-checks
 * (src/ffi/qsfi.rs:472-516,539-587). */
qsfi_status
qsfi_moe_plan_create(qsfi_context* ctx, const qsfi_moe_plan_desc* desc, qsfi_moe_plan** out);
void qsfi_moe_plan_destroy(qsfi_moe_plan* plan);
qsfi_status qsfi_moe_workspace_size(
    qsfi_context* ctx, const qsfi_moe_plan* plan, uint32_t num_tokens, size_t* device_bytes
);
qsfi_status qsfi_moe_execute_bf16(
    qsfi_context* ctx, const qsfi_moe_plan* plan, const qsfi_moe_bf16_execute_desc* desc
);
qsfi_status qsfi_moe_execute_nvfp4(
    qsfi_context* ctx, const qsfi_moe_plan* plan, const qsfi_moe_nvfp4_execute_desc* desc
);

/* ------------------------------------------------- router & glue (qscu) -- */

typedef enum { /* upstream qscu.h:202 */
    QSCU_ROUTER_SCORE_SOFTMAX = 0,
    QSCU_ROUTER_SCORE_SIGMOID = 1
} qscu_router_score;

typedef struct { /* upstream qscu.h:246-256 */
    qsfi_tensor2 logits;       /* bf16/f32 [num_tokens, num_experts] */
    qsfi_tensor2 topk_ids;     /* i32 [num_tokens, top_k], descending score, ties by lower id */
    qsfi_tensor2 topk_weights; /* f32 [num_tokens, top_k] */
    uint32_t num_tokens;
    uint32_t num_experts; /* <= 4096 */
    uint32_t top_k;       /* <= 16 and <= num_experts */
    qscu_router_score score;
    uint32_t renormalize;
    float routed_scaling_factor; /* finite, > 0 */
} qscu_router_topk_desc;

/* Softmax/sigmoid top-k routing, upstream qscu.h:278 (qscu.cu:894-971,1817-1857).
 * One warp per token instead of upstream's one thread per token; the selection
 * order, tie-break, NaN handling and renormalisation are upstream's. */
qsfi_status qscu_router_topk(const qscu_router_topk_desc* desc, qsfi_cuda_stream stream);

typedef struct { /* upstream qscu.h:27-33 */
    qsfi_tensor2 gate;
    qsfi_tensor2 up;
    qsfi_tensor2 out;
    uint32_t num_tokens;
    uint32_t intermediate_size;
} qscu_silu_and_mul_desc;

/* out = silu(gate) * up on bf16 rows, upstream qscu.h:35 (qscu.cu:306-327). */
qsfi_status qscu_silu_and_mul_bf16(const qscu_silu_and_mul_desc* desc, qsfi_cuda_stream stream);

typedef struct { /* upstream qscu.h:42-48 */
    qsfi_tensor2 gate_logits; /* bf16/f32 [num_tokens, 1] */
    qsfi_tensor2 shared;      /* bf16 [num_tokens, hidden] */
    qsfi_tensor2 out;         /* bf16 [num_tokens, hidden], updated in place */
    uint32_t num_tokens;
    uint32_t hidden_size;
} qscu_qwen36_shared_expert_gate_add_desc;

/* out += sigmoid(gate_logits[t]) * shared, upstream qscu.h:50-52 (qscu.cu:338-355). */
qsfi_status qscu_qwen36_shared_expert_gate_add_bf16(
    const qscu_qwen36_shared_expert_gate_add_desc* desc, qsfi_cuda_stream stream
);

/* ------------------------------------------------ dense bf16 GEMM (qscb) -- */

typedef struct qscb_context qscb_context; /* upstream qscb.h:27 */

typedef struct { /* upstream qscb.h:29-32 */
    int32_t device_ordinal;
    qsfi_cuda_stream stream;
} qscb_context_desc;

typedef struct { /* upstream qscb.h:34-45 */
    qsfi_tensor2 x;      /* bf16 [rows, in_features], stride[1] == 1, padded rows allowed */
    qsfi_tensor2 weight; /* bf16 [out_features, in_features] */
    qsfi_tensor2 out;    /* bf16 or f32 [rows, out_features] */
    uint32_t rows;
    uint32_t in_features;
    uint32_t out_features;
    float alpha; /* 0 means 1 */
    float beta;
    qsfi_device_ptr workspace; /* unused by this build */
    size_t workspace_bytes;
} qscb_bf16_gemm_desc;

/* out = alpha * x * weight^T + beta * out with f32 accumulation, upstream
 * qscb.h:47-52 (qscb.cu:265-470). The router-logits GEMM and the shared-expert
 * projections of the MoE layer go through this call (src/model.rs:2082-2090,
 * 2184-2226). tcgen05 kind::f16 kernel; no cuBLASLt. */
qsfi_status qscb_context_create(const qscb_context_desc* desc, qscb_context** out);
void qscb_context_destroy(qscb_context* ctx);
qsfi_status qscb_context_get_last_error(const qscb_context* ctx, qsfi_error_info* out);
void qscb_context_clear_last_error(qscb_context* ctx);
qsfi_status qscb_gemm_bf16(qscb_context* ctx, const qscb_bf16_gemm_desc* desc);

/* ---- RMSNorm neighbours of the MoE block (upstream qsfi.h:160-176, 330-331; there a
 * FlashInfer call, qsfi_norm_rope.cu:139-206, 395-465). Same descriptors, validation
 * order and messages (qsfi_norm_rope.cu:72-146, 208-238). ---- */
typedef struct {
    qsfi_tensor2 x;      /* bf16/f32 [rows, hidden_size]. */
    qsfi_tensor1 weight; /* same dtype [hidden_size]. */
    qsfi_tensor2 out;    /* same dtype [rows, hidden_size]. */
    uint32_t hidden_size;
    float weight_bias;   /* 0 for standard RMSNorm, 1 for raw-weight+1 q/k norm. */
    float eps;
} qsfi_rmsnorm_desc;

typedef struct {
    qsfi_tensor2 x;              /* bf16/f32 [rows, hidden_size], overwritten with normalized output. */
    qsfi_tensor2 residual_inout; /* same dtype [rows, hidden_size], updated to residual + x. */
    qsfi_tensor1 weight;         /* same dtype [hidden_size]. */
    qsfi_tensor2 out;            /* must alias x; documents the normalized output tensor. */
    uint32_t hidden_size;
    float eps;
} qsfi_fused_add_rmsnorm_desc;

qsfi_status qsfi_rmsnorm(qsfi_context* ctx, const qsfi_rmsnorm_desc* desc);
qsfi_status qsfi_fused_add_rmsnorm(qsfi_context* ctx, const qsfi_fused_add_rmsnorm_desc* desc);

/* ============================ additive entry points (no upstream symbol) == */

/* Scale-factor tile layout used by the block-scaled tensor-core path
 * ("tiled"): scales of a [rows, K] operand with one e4m3 scale per 16 elements
 * are stored per (128-row block, 64-element k group) as a 512-byte tile,
 *   byte = ((row_block * (K/64) + k_group) * 512) + (row % 32) * 16
 *          + ((row / 32) % 4) * 4 + (k / 16) % 4,
 * which is what one tcgen05.cp 32x128b.warpx4 moves into tensor memory. */

/* Returns the number of bytes of the tiled scale buffer for a [rows, k] operand. */
size_t qs3_nvfp4_tiled_scale_bytes(uint64_t rows, uint64_t k);

typedef struct {
    qsfi_tensor3 weight;        /* bf16 [experts, rows, k], contiguous */
    qsfi_tensor3 packed;        /* u8 [experts, rows, k/2] out */
    qsfi_tensor3 scale_linear;  /* optional e4m3 [experts, rows, k/16] out (declared ABI layout) */
    qsfi_tensor1 scale_tiled;   /* optional u8 [experts * qs3_nvfp4_tiled_scale_bytes(rows,k)] out */
    qsfi_tensor1 global_scale;  /* f32 [experts] out: amax / (6 * 448), 1 when amax == 0 */
    uint32_t gated_rows;        /* != 0: rows = 2*inter (gate rows then up rows); the tiled scale
                                   buffer then interleaves 64 gate rows with their 64 up rows per
                                   128-row block, matching the gate_up GEMM tile */
} qs3_nvfp4_quantize_weight_desc;

/* Quantise bf16 expert weights to NVFP4 (e2m1 codes, one e4m3 scale per 16
 * elements along k, one f32 scale per expert). Stands in for the quantised
 * layout the upstream weight loader never produced (src/weight_loader.rs:33-66,
 * AGENTS.md:45-47). */
qsfi_status qs3_nvfp4_quantize_weight(qsfi_context* ctx, const qs3_nvfp4_quantize_weight_desc* desc);

typedef struct {
    qsfi_tensor2 x;            /* bf16 [rows, k] */
    qsfi_tensor2 packed;       /* u8 [rows, k/2] out */
    qsfi_tensor2 scale_linear; /* e4m3 [rows, k/16] out */
    float global_scale;        /* 0 means 1 */
    uint32_t rows;
} qs3_nvfp4_quantize_act_desc;

/* Quantise bf16 activation rows to the declared NVFP4 activation layout
 * (hidden_packed / hidden_scale of qsfi_moe_nvfp4_execute_desc). */
qsfi_status qs3_nvfp4_quantize_act(qsfi_context* ctx, const qs3_nvfp4_quantize_act_desc* desc);

/* Re-tile declared-layout ("linear") weight scales into the tiled layout once,
 * so that execute calls need not do it per call. */
typedef struct {
    qsfi_tensor3 scale_linear; /* e4m3 [experts, rows, k/16] */
    qsfi_tensor1 scale_tiled;  /* u8 out */
    uint32_t gated_rows;
} qs3_nvfp4_tile_scales_desc;
qsfi_status qs3_nvfp4_tile_scales(qsfi_context* ctx, const qs3_nvfp4_tile_scales_desc* desc);

/* Fused add + RMSNorm (bf16) that also writes the NVFP4 quantisation of the normalised rows
 * in token order (codes + tiled scales): the pre-MoE norm then hands the MoE layer its
 * tokens already quantised, in the same pass over [rows, hidden]. No upstream counterpart.
 * The codes equal qs3_nvfp4_quantize_act applied to the bf16 rows this call stores. */
typedef struct {
    qsfi_fused_add_rmsnorm_desc norm; /* bf16, hidden_size divisible by 64 and <= 8192 */
    qsfi_tensor2 packed;              /* u8 [rows, hidden_size / 2] out */
    qsfi_tensor1 scale_tiled;         /* u8 [>= qs3_nvfp4_tiled_scale_bytes(rows, hidden_size)] out */
    float global_scale;               /* 0 means 1 */
} qs3_fused_add_rmsnorm_nvfp4_desc;
qsfi_status qs3_fused_add_rmsnorm_nvfp4(qsfi_context* ctx, const qs3_fused_add_rmsnorm_nvfp4_desc* desc);

/* ---- FP8 block-scaled experts (no upstream counterpart: upstream declares only the
 * dtype values QSFI_DTYPE_FP8_E4M3 / _E5M2, qs_tensor.h:20-24, and no FP8 MoE entry) ----
 * Weights: e4m3 codes [experts, rows, k] with one f32 scale per 128 x 128 block,
 * scale tensor f32 [experts, ceil(rows / 128), k / 128]. Activations: e4m3 codes
 * [tokens, k] with one f32 scale per token per 128 elements, f32 [tokens, k / 128].
 *   scale = max(amax / 448, 1e-30),  code = e4m3_rn_sat(x * (1 / scale)).
 * A plan for this path has backend = QS3_MOE_BACKEND_FP8_BLOCKSCALE, activation and
 * weight dtype QSFI_DTYPE_FP8_E4M3, output dtype bf16; hidden_size and
 * intermediate_size must be multiples of 128 and at most 4096. */
#define QS3_MOE_BACKEND_FP8_BLOCKSCALE 100

typedef struct {
    qsfi_tensor3 weight; /* bf16 [experts, rows, k], contiguous */
    qsfi_tensor3 codes;  /* e4m3 [experts, rows, k] out */
    qsfi_tensor3 scale;  /* f32 [experts, ceil(rows / 128), k / 128] out */
} qs3_fp8_quantize_weight_desc;
qsfi_status qs3_fp8_quantize_weight(qsfi_context* ctx, const qs3_fp8_quantize_weight_desc* desc);

typedef struct {
    qsfi_tensor2 x;     /* bf16 [rows, k] */
    qsfi_tensor2 codes; /* e4m3 [rows, k] out */
    qsfi_tensor2 scale; /* f32 [rows, k / 128] out */
    uint32_t rows;
} qs3_fp8_quantize_act_desc;
qsfi_status qs3_fp8_quantize_act(qsfi_context* ctx, const qs3_fp8_quantize_act_desc* desc);

/* Routed experts on FP8 operands with precomputed routing: the FP8 sibling of
 * qsfi_moe_execute_nvfp4 (same roles of the tensors, same workspace query
 * qsfi_moe_workspace_size). SwiGLU output is re-quantised per token per 128
 * features before the down projection. No counterpart in the reference: its
 * qsfi.h has no FP8 MoE entry (backends 1..3, qsfi.h:206-209), hence the qs3_
 * prefix. The names qsfi_moe_execute_fp8 / qsfi_moe_fp8_execute_desc of earlier
 * versions of this header stay as aliases. */
typedef struct {
    qsfi_tensor2 hidden;               /* e4m3 [num_tokens, hidden] */
    qsfi_tensor2 hidden_scale;         /* f32 [num_tokens, hidden / 128] */
    qsfi_tensor2 topk_ids;             /* i32 [num_tokens, top_k] */
    qsfi_tensor2 topk_weights;         /* f32 [num_tokens, top_k] */
    qsfi_tensor3 gate_up_weight;       /* e4m3 [E_local, 2I, H] */
    qsfi_tensor3 gate_up_weight_scale; /* f32 [E_local, 2I / 128, H / 128] */
    qsfi_tensor3 down_weight;          /* e4m3 [E_local, H, I] */
    qsfi_tensor3 down_weight_scale;    /* f32 [E_local, H / 128, I / 128] */
    qsfi_tensor2 out;                  /* bf16 [num_tokens, hidden] */
    qsfi_tensor1 workspace;            /* u8 [>= qsfi_moe_workspace_size] */
    uint32_t num_tokens;
} qs3_moe_fp8_execute_desc;
typedef qs3_moe_fp8_execute_desc qsfi_moe_fp8_execute_desc;
qsfi_status qs3_moe_execute_fp8(qsfi_context* ctx, const qsfi_moe_plan* plan, const qs3_moe_fp8_execute_desc* desc);
qsfi_status
qsfi_moe_execute_fp8(qsfi_context* ctx, const qsfi_moe_plan* plan, const qsfi_moe_fp8_execute_desc* desc);

/* Whole MoE layer in one call: what upstream's execute_moe_mlp issues as five
 * GEMM calls, a router call, a MoE call and two element-wise calls
 * (src/model.rs:2072-2228), i.e. the QSFI_MOE_ROUTE_ROUTER_LOGITS mode upstream
 * declares but rejects (qsfi_moe.cu:157-159). */
typedef struct {
    /* inputs */
    qsfi_tensor2 hidden;        /* bf16 [num_tokens, hidden] */
    qsfi_tensor2 router_weight; /* bf16 [num_experts, hidden] */
    qsfi_tensor1 router_bias;   /* optional f32 [num_experts], added to the logits before top-k */
    /* routed experts: bf16 plan -> *_weight bf16; NVFP4 plan -> packed + tiled scales;
       FP8 plan -> e4m3 codes [E_local, 2I, H] / [E_local, H, I], and the *_scale_tiled
       fields carry the f32 block scales as flat f32 tensors
       ([E_local * (2I / 128) * (H / 128)] and [E_local * (H / 128) * (I / 128)]);
       FP8 plans take no shared expert */
    qsfi_tensor3 gate_up_weight;       /* bf16 [E_local, 2I, H] or u8 [E_local, 2I, H/2] */
    qsfi_tensor1 gate_up_scale_tiled;  /* NVFP4 / FP8 only */
    qsfi_tensor1 gate_up_global_scale; /* NVFP4 only, f32 [E_local], or f32 [2 * E_local]: the global
                                          scales of the gate rows followed by those of the up rows
                                          (checkpoints that quantise gate_proj and up_proj apart) */
    qsfi_tensor3 down_weight;          /* bf16 [E_local, H, I] or u8 [E_local, H, I/2] */
    qsfi_tensor1 down_scale_tiled;     /* NVFP4 / FP8 only */
    qsfi_tensor1 down_global_scale;    /* NVFP4 only, f32 [E_local] */
    /* optional shared expert (data == NULL on shared_gate_up_weight: none); same dtype family */
    qsfi_tensor3 shared_gate_up_weight;       /* [1, 2*Is, H] (or packed) */
    qsfi_tensor1 shared_gate_up_scale_tiled;
    qsfi_tensor1 shared_gate_up_global_scale; /* f32 [1], or f32 [2]: gate rows, up rows */
    qsfi_tensor3 shared_down_weight;          /* [1, H, Is] (or packed) */
    qsfi_tensor1 shared_down_scale_tiled;
    qsfi_tensor1 shared_down_global_scale;    /* f32 [1] */
    qsfi_tensor2 shared_gate_weight;          /* bf16 [1, hidden]: sigmoid gate logit row */
    uint32_t shared_intermediate_size;
    /* routing parameters (upstream src/lib.rs:21-24 uses softmax, renormalise, 1.0) */
    qscu_router_score score;
    uint32_t renormalize;
    float routed_scaling_factor;
    float act_global_scale;  /* NVFP4: global scale of the hidden activations, 0 means 1 */
    float act2_global_scale; /* NVFP4: global scale of the SwiGLU output, 0 means 1 */
    /* outputs */
    qsfi_tensor2 out;          /* bf16 [num_tokens, hidden] */
    qsfi_tensor2 topk_ids;     /* optional i32 [num_tokens, top_k] out */
    qsfi_tensor2 topk_weights; /* optional f32 [num_tokens, top_k] out */
    qsfi_tensor2 router_logits; /* optional f32 [num_tokens, num_experts] out */
    qsfi_tensor1 workspace;    /* u8 [>= qs3_moe_layer_workspace_size] */
    uint32_t num_tokens;
    /* optional, NVFP4 plans: the tokens already quantised in token order (codes u8
       [num_tokens, hidden / 2] and tiled scales covering ceil(num_tokens / 128) * 128 rows),
       as qs3_fused_add_rmsnorm_nvfp4 writes them with the same act_global_scale; the layer
       then skips its own quantisation pass. `hidden` is still needed (router, shared gate). */
    qsfi_tensor2 hidden_packed;
    qsfi_tensor1 hidden_scale_tiled;
    /* optional: the block's post-MoE neighbours fused into the combine (hidden <= 2048):
       residual_inout (bf16 [num_tokens, hidden], contiguous) += the layer's output, in place,
       and `out` receives rmsnorm(residual_inout) * next_norm_weight instead of the raw MoE
       output, i.e. qsfi_fused_add_rmsnorm applied to the layer's output in the same pass. */
    qsfi_tensor2 residual_inout;
    qsfi_tensor1 next_norm_weight; /* bf16 [hidden] */
    float next_norm_eps;
} qs3_moe_layer_desc;

qsfi_status qs3_moe_layer_workspace_size(
    qsfi_context* ctx, const qsfi_moe_plan* plan, uint32_t num_tokens,
    uint32_t shared_intermediate_size, size_t* device_bytes
);
qsfi_status
qs3_moe_layer_execute(qsfi_context* ctx, const qsfi_moe_plan* plan, const qs3_moe_layer_desc* desc);

/* ---- expert parallelism (no upstream counterpart: upstream rejects partial expert ranges) ----
 * One layer on n ranks, experts split in contiguous blocks, tokens data-parallel:
 *   qs3_moe_ep_route            local tokens -> top-k ids/weights (+ NVFP4 codes of the tokens)
 *   [caller: all-gather of codes, scales, ids, weights over NCCL]
 *   qs3_moe_execute_nvfp4_prepared   local experts over ALL gathered tokens -> partial sums
 *   [caller: all-to-all of the partial sums back to the token owners over NCCL]
 *   qs3_moe_ep_finish           shared expert + sum of the n partials in rank order -> out
 * The exchanges belong to the caller; the library never waits on another rank. */
typedef struct {
    qsfi_tensor2 hidden;         /* in:  bf16 [num_tokens, hidden] */
    qsfi_tensor2 router_weight;  /* in:  bf16 [num_experts, hidden] */
    qsfi_tensor1 router_bias;    /* in:  optional f32 [num_experts] */
    qsfi_tensor2 router_logits;  /* out: f32 [num_tokens, num_experts] (scratch the caller owns) */
    qsfi_tensor2 topk_ids;       /* out: i32 [num_tokens, top_k], global ids */
    qsfi_tensor2 topk_weights;   /* out: f32 [num_tokens, top_k] */
    qsfi_tensor2 hidden_packed;  /* out, optional: u8 [num_tokens, hidden/2] */
    qsfi_tensor2 hidden_scale;   /* out, with hidden_packed: e4m3 [num_tokens, hidden/16], linear */
    qscu_router_score score;
    uint32_t renormalize;
    float routed_scaling_factor;
    float act_global_scale;      /* 0 means 1 */
    uint32_t num_tokens;
    /* Optional: placements with replicated experts. The plan then counts expert SLOTS (every rank
       holds its own experts plus replicas of the hottest ones: num_experts = ranks * slots per rank)
       while the router still scores the model's experts: router_weight / router_bias /
       router_logits have expert_id_map.shape[0] rows / entries / columns instead of
       plan.num_experts, topk_ids receives the router's expert ids, and dispatch_ids[t, k] =
       expert_id_map[topk_ids[t, k]] the slot each route goes to (on this rank: a hot expert maps
       to this rank's own replica). dispatch_ids is what the other phases take as topk_ids. */
    qsfi_tensor1 expert_id_map;  /* in:  optional i32 [router experts] */
    qsfi_tensor2 dispatch_ids;   /* out: with expert_id_map: i32 [num_tokens, top_k] */
    /* Optional: rank_mask[t] = the set of ranks token t has a route to (bit r: one of its dispatch ids
       lies in rank r's plan.local_num_experts slots), for a dispatch that moves a token only to the
       ranks that need it (qs3_moe_ep_pull_routed). */
    qsfi_tensor1 rank_mask;      /* out: optional u32 (dtype I32) [num_tokens] */
    uint32_t num_ranks;          /* with rank_mask */
} qs3_moe_ep_route_desc;
qsfi_status qs3_moe_ep_route(qsfi_context* ctx, const qsfi_moe_plan* plan, const qs3_moe_ep_route_desc* desc);

/* qsfi_moe_execute_nvfp4 with prepared weights: activations in the declared layout
 * (linear scales), weights as qs3_nvfp4_quantize_weight leaves them (tiled scales +
 * per-expert global scales). Workspace: qsfi_moe_workspace_size of the plan suffices. */
typedef struct {
    qsfi_tensor2 hidden_packed;        /* u8   [num_tokens, hidden/2] */
    qsfi_tensor2 hidden_scale;         /* e4m3 [num_tokens, hidden/16] */
    qsfi_tensor2 topk_ids;             /* i32  [num_tokens, top_k], global ids */
    qsfi_tensor2 topk_weights;         /* f32  [num_tokens, top_k] */
    qsfi_tensor3 gate_up_weight;       /* u8   [local_experts, 2*inter, hidden/2] */
    qsfi_tensor1 gate_up_scale_tiled;
    qsfi_tensor1 gate_up_global_scale; /* optional f32 [local_experts] or [2 * local_experts] (gate, up) */
    qsfi_tensor3 down_weight;          /* u8   [local_experts, hidden, inter/2] */
    qsfi_tensor1 down_scale_tiled;
    qsfi_tensor1 down_global_scale;    /* optional f32 [local_experts] */
    float act_global_scale;
    float act2_global_scale;
    qsfi_tensor2 out;                  /* bf16 [num_tokens, hidden]: sum over the LOCAL routes */
    qsfi_tensor1 workspace;
    uint32_t num_tokens;
    uint32_t flags; /* bit 0: leave `out` rows of tokens that have no local route unwritten */
} qs3_moe_nvfp4_prepared_desc;
qsfi_status qs3_moe_execute_nvfp4_prepared(
    qsfi_context* ctx, const qsfi_moe_plan* plan, const qs3_moe_nvfp4_prepared_desc* desc
);

typedef struct {
    qsfi_tensor2 hidden;                      /* bf16 [num_tokens, hidden], this rank's tokens */
    qsfi_tensor3 partials;                    /* bf16 [num_ranks, num_tokens, hidden] (phase 2) */
    qsfi_tensor3 shared_gate_up_weight;       /* optional shared expert, NVFP4 as in qs3_moe_layer_desc */
    qsfi_tensor1 shared_gate_up_scale_tiled;
    qsfi_tensor1 shared_gate_up_global_scale;
    qsfi_tensor3 shared_down_weight;
    qsfi_tensor1 shared_down_scale_tiled;
    qsfi_tensor1 shared_down_global_scale;
    qsfi_tensor2 shared_gate_weight;
    uint32_t shared_intermediate_size;
    float act_global_scale;
    float act2_global_scale;
    qsfi_tensor2 out;                         /* bf16 [num_tokens, hidden] (phase 2) */
    qsfi_tensor1 workspace;                   /* >= qs3_moe_ep_finish_workspace_size; keep it between phases */
    uint32_t num_tokens;
    uint32_t num_ranks;
    uint32_t phases; /* bit 0: shared expert (can run while the exchange is in flight); bit 1: sum + store */
    /* Pull mode of phase 2 (peer_partials != NULL, `partials` unused): instead of summing
     * exchanged copies, read every rank's partial-sum buffer [num_ranks * num_tokens, hidden]
     * in place through peer-mapped pointers (HOST array of num_ranks device pointers, entry r
     * = rank r's buffer as mapped on this device). Only (token, rank) pairs that have a route
     * are read, decided from this rank's own topk_ids and the plan's expert block
     * (rank r owns experts [r * local_num_experts, (r + 1) * local_num_experts)). The caller
     * orders the launch after every rank finished writing its buffer (a barrier or any
     * collective on the stream) and does not let a rank overwrite it before all ranks ran
     * this phase. */
    const qsfi_device_ptr* peer_partials;
    qsfi_tensor2 topk_ids; /* i32 [num_tokens, top_k], pull mode only */
} qs3_moe_ep_finish_desc;
qsfi_status qs3_moe_ep_finish_workspace_size(
    qsfi_context* ctx, const qsfi_moe_plan* plan, uint32_t num_tokens, uint32_t num_ranks,
    uint32_t shared_intermediate_size, size_t* device_bytes
);
qsfi_status qs3_moe_ep_finish(qsfi_context* ctx, const qsfi_moe_plan* plan, const qs3_moe_ep_finish_desc* desc);

/* Dispatch by pulling: every rank keeps the outputs of qs3_moe_ep_route (codes, scales, ids,
 * weights of its own tokens) in one peer-mapped block; this call copies up to four
 * segments of the blocks of ALL ranks into local buffers laid out [num_ranks, segment] with
 * plain peer loads over NVLink, i.e. an all-gather without a collective library. The
 * caller orders it after every rank finished writing its block (a barrier on the stream)
 * and does not let a rank overwrite its block before all ranks ran this call. */
typedef struct {
    const qsfi_device_ptr* peer_blocks; /* [num_ranks] base of rank r's block as mapped on this device */
    uint64_t segment_offset[4];         /* byte offset of segment j inside a block, multiple of 16 */
    uint64_t segment_bytes[4];          /* bytes of segment j per rank, multiple of 16 */
    qsfi_device_ptr dst[4];             /* local destination of segment j, num_ranks * segment_bytes[j] bytes */
    uint32_t num_ranks;                 /* <= 32 */
    uint32_t num_segments;              /* <= 4 */
} qs3_moe_ep_pull_tokens_desc;
qsfi_status qs3_moe_ep_pull_tokens(qsfi_context* ctx, const qs3_moe_ep_pull_tokens_desc* desc);

/* De-duplicated dispatch by pulling. Every rank keeps, in one peer-mapped block, the outputs of
 * qs3_moe_ep_route for its own tokens: codes, linear scales, dispatch ids, weights and the rank
 * mask. This call fills the local [num_ranks * num_tokens, ...] buffers: ids and weights of every
 * token of every rank (the route sort needs them), codes and scales only of the tokens whose mask
 * has this rank's bit, i.e. each token row crosses NVLink once per rank that holds one of its
 * experts and not at all otherwise. Rows that are not pulled are left as they were. Ordering
 * against the other ranks as for qs3_moe_ep_pull_tokens (qs3_moe_ep_barrier before and after). */
typedef struct {
    const qsfi_device_ptr* peer_blocks; /* [num_ranks] base of rank r's block as mapped on this device */
    uint64_t offset_codes, offset_scales, offset_ids, offset_weights, offset_mask; /* in a block, 16-byte aligned */
    qsfi_device_ptr dst_codes;   /* u8  [num_ranks * num_tokens, hidden / 2] */
    qsfi_device_ptr dst_scales;  /* e4m3 [num_ranks * num_tokens, hidden / 16] */
    qsfi_device_ptr dst_ids;     /* i32 [num_ranks * num_tokens, top_k] */
    qsfi_device_ptr dst_weights; /* f32 [num_ranks * num_tokens, top_k] */
    uint32_t num_ranks;          /* <= 32 */
    uint32_t my_rank;
    uint32_t num_tokens;         /* per rank */
    uint32_t top_k;              /* <= 16 */
    uint32_t hidden_size;        /* multiple of 256, <= 2048 */
} qs3_moe_ep_pull_routed_desc;
qsfi_status qs3_moe_ep_pull_routed(qsfi_context* ctx, const qs3_moe_ep_pull_routed_desc* desc);

/* Barrier over the ranks of an expert-parallel layer, on the context's stream, without a
 * collective library: every rank owns a signal pad of num_ranks u32 words in peer-mapped memory
 * (zeroed once); the kernel stores `epoch` into its slot of every rank's pad and waits until every
 * slot of its own pad has reached `epoch` (plain release stores / acquire loads at system scope
 * over NVLink). `epoch` must grow by one with every barrier on the same pads. With `epoch_counter`
 * (a u32 in this rank's own device memory, zeroed once) the kernel takes epoch = counter + 1 and
 * stores it back, so the launch carries no per-step argument and a whole step can be replayed from
 * a CUDA graph; every rank must then run the same sequence of barriers. The wait is bounded:
 * after timeout_cycles SM clocks (0: about two seconds) the kernel records a code in the device
 * error word and returns, so a rank that died or never got here turns into
 * QSFI_STATUS_BACKEND_ERROR at the next qs3_moe_check_device_error instead of a hung GPU. */
typedef struct {
    const qsfi_device_ptr* pads; /* [num_ranks] rank r's pad as mapped on this device */
    uint32_t num_ranks;          /* <= 32 */
    uint32_t my_rank;
    uint32_t epoch;              /* ignored when epoch_counter is set */
    uint64_t timeout_cycles;
    qsfi_device_ptr epoch_counter; /* optional u32 [1], 4-byte aligned */
} qs3_moe_ep_barrier_desc;
qsfi_status qs3_moe_ep_barrier(qsfi_context* ctx, const qs3_moe_ep_barrier_desc* desc);

/* Synchronises the context's stream and turns a recorded bounded-wait expiry (see
 * qs3_moe_read_device_error) into QSFI_STATUS_BACKEND_ERROR with the code in the last-error
 * message; QSFI_STATUS_OK when nothing expired. Clears the error word. */
qsfi_status qs3_moe_check_device_error(qsfi_context* ctx);

/* Test aid: launches one small kernel whose threads wait on an mbarrier that nothing ever
 * completes, with `limit_cycles` (1 .. 2e7 SM clocks) as the wait limit. The kernel must return
 * after about that many clocks with the expiry code in the device error word. Nothing faults,
 * traps or hangs; this exercises the path every bounded wait of the tensor-core kernels takes
 * when its producer is lost. */
qsfi_status qs3_debug_bounded_wait_probe(qsfi_context* ctx, uint64_t limit_cycles);

/* Measurement aids of the CTA-pair GEMM (gemm_pair.cu), filled when QS3_PAIR_DBG has bit 32 set:
 * clock64() stamps of the first cluster's producer / scale copier / MMA issuer / epilogue warp 0 at
 * their hand-over points ([4 roles][192 stages][4 events]), and per cluster the global-timer
 * start / end (ns) and unit count of its MMA issuer ([128][3]). */
qsfi_status qs3_debug_pair_trace(uint64_t* out, uint32_t capacity, uint32_t* count);
qsfi_status qs3_debug_pair_spans(uint64_t* out, uint32_t capacity);

/* Routing tables of the last execute on this workspace, for parity checks:
 * copies of counts[E_local], indptr[E_local+1], route_rows[T*K] (-1: not local),
 * row_tokens[R_local], row_scales[R_local] (upstream qsfi_moe.cu:26-31). Device
 * pointers into `workspace`; valid until the next execute on it. */
typedef struct {
    const int32_t* counts;
    const int32_t* indptr;
    const int32_t* route_rows;
    const int32_t* row_tokens;
    const float* row_scales;
} qs3_moe_routing_view;
qsfi_status qs3_moe_routing_tables(
    qsfi_context* ctx, const qsfi_moe_plan* plan, uint32_t num_tokens, qsfi_device_ptr workspace,
    qs3_moe_routing_view* out
);

/* Route sort that allocates nothing. No counterpart in the reference: upstream only
 * ever sorts routes inside qsfi_moe_execute_bf16 with scratch from the caller's
 * workspace. This entry point is for callers that cannot allocate device memory when
 * they need the routing tables (all HBM already committed to fixed pools at start-up,
 * or a section where cudaMalloc's device-wide synchronisation is unacceptable): the
 * kernels' scratch lives in a fixed QS3_ROUTE_SORT_STATIC_SCRATCH_BYTES array inside
 * the library image, which every GPU that loads the library keeps until exit.
 *
 *  - Inputs and outputs are still the caller's: topk_ids / topk_weights in; counts,
 *    indptr, route_rows (-1 for routes to non-local experts), row_tokens, row_scales
 *    out, identical to what qs3_moe_routing_tables reports after an execute call.
 *  - Limits: num_tokens * top_k <= QS3_ROUTE_SORT_STATIC_MAX_ROUTES and
 *    local_num_experts <= QS3_ROUTE_SORT_STATIC_MAX_EXPERTS; anything larger returns
 *    QSFI_STATUS_UNSUPPORTED with the limits in the context's last-error message.
 *  - No cudaMalloc, cudaFree or allocating library routine is called. The first call on
 *    each device resolves the array's device address (cudaGetSymbolAddress); make that
 *    first call before starting any stream capture on that device.
 *  - All calls on one device share the one array and it keeps the previous call's
 *    contents. Nothing in it has to start at zero (every word is written before it is
 *    read within a call), but two calls whose kernels overlap on the GPU (different
 *    streams, or different host threads) race on it: serialise them. */
#define QS3_ROUTE_SORT_STATIC_MAX_ROUTES 131072u
#define QS3_ROUTE_SORT_STATIC_MAX_EXPERTS 1024u
#define QS3_ROUTE_SORT_STATIC_SCRATCH_BYTES (2u << 20)
typedef struct {
    qsfi_tensor2 topk_ids;     /* in:  i32 [num_tokens, top_k], global expert ids */
    qsfi_tensor2 topk_weights; /* in:  f32 [num_tokens, top_k] */
    qsfi_tensor1 counts;       /* out: i32 [>= local_num_experts] */
    qsfi_tensor1 indptr;       /* out: i32 [>= local_num_experts + 1] */
    qsfi_tensor1 route_rows;   /* out: i32 [>= num_tokens * top_k] */
    qsfi_tensor1 row_tokens;   /* out: i32 [>= num_tokens * top_k], first indptr[E] entries valid */
    qsfi_tensor1 row_scales;   /* out: f32 [>= num_tokens * top_k], first indptr[E] entries valid */
    uint32_t num_tokens;
    uint32_t top_k;
    uint32_t local_expert_offset;
    uint32_t local_num_experts;
} qs3_route_sort_static_desc;
qsfi_status qs3_moe_route_sort_static(qsfi_context* ctx, const qs3_route_sort_static_desc* desc);

/* Device-side error word of the tensor-core kernels: every wait inside them is
 * bounded; a wait that runs out records where and the kernel returns. Reads
 * (and clears) the word; synchronises the context's stream. 0 = no error. */
qsfi_status qs3_moe_read_device_error(qsfi_context* ctx, uint32_t* code);

/* Measurement aids. qs3_moe_launch_count: kernels this library has launched in this
 * process so far. qs3_moe_profile_begin / _end: between the two calls every
 * qs3_moe_layer_execute records a CUDA event on the context's stream at each stage
 * boundary; _end synchronises the stream and returns, per recorded stage, its id
 * (1 router-logits GEMM, 2 router top-k, 3 route sort, 4 gather/quantise, 5 gate_up
 * GEMM + SwiGLU, 6 down GEMM, 7 shared expert, 8 combine) and its duration in ms. */
uint64_t qs3_moe_launch_count(void);
qsfi_status qs3_moe_profile_begin(qsfi_context* ctx);
qsfi_status qs3_moe_profile_end(
    qsfi_context* ctx, int32_t* stage_ids, float* stage_ms, uint32_t capacity, uint32_t* count
);

/* Tensor-pipe ceiling of one tcgen05.mma shape on the context's device, no counterpart
 * upstream: every SM issues `iters` x 4 back-to-back 128 x n MMAs (K = 32 bytes each) on
 * operands resident in shared memory, timed with CUDA events on the context's stream.
 * kind 0 = bf16 (kind::f16), 1 = fp8 e4m3 (kind::f8f6f4), 2 = NVFP4 block-scaled
 * (kind::mxf4nvf4, scale_vec::4X). n is a multiple of 16 in [16, 256]. kind + 16: CTA
 * pairs (clusters of two) issue cta_group::2 instructions of 256 x n instead (n a multiple
 * of 32). kind + 256 * a + 4096 * b (single-CTA NVFP4 probe only, a, b <= 8): every iteration
 * also issues a scale-tile copies (tcgen05.cp, 512 bytes each) from the MMA thread ahead of its
 * MMAs and b from a second thread, which measures what the scale copies of a block-scaled
 * main loop cost. Returns dense TFLOP/s. Used as the denominator of the reported
 * tensor-pipe fractions. */
qsfi_status qs3_tensor_peak_probe(qsfi_context* ctx, uint32_t kind, uint32_t n, uint32_t iters, double* tflops);

/* Operand-delivery ceiling (L2 -> shared memory) on the context's device, no counterpart upstream:
 * every SM streams `tiles` tiles of `tile_bytes` out of `buffer` into its shared memory with bulk
 * copies (cp.async.bulk, the path the GEMM operands take), `stages` of them in flight, and discards
 * them; a first untimed pass fills the L2 when the buffer fits it. pattern 0: tiles are contiguous
 * (operands stored as shared-memory images); pattern 1: a tile is a 128-row x 128-byte swizzled box
 * of a matrix with 1 KiB rows (tile_bytes 16384, cp.async.bulk.tensor). Returns GB/s over all SMs. The
 * grouped NVFP4 GEMMs stream their weights once per pair of row tiles; this is the rate that stream
 * can reach for a given number of bytes in flight. */
qsfi_status qs3_operand_stream_probe(qsfi_context* ctx, qsfi_device_ptr buffer, uint64_t buffer_bytes,
                                     uint32_t tile_bytes, uint32_t stages, uint32_t tiles, uint32_t pattern,
                                     double* gbs);

/* ================================================= checkpoint loader ======
 * Upstream has the loader only as a trait (src/weight_loader.rs:33-38: alloc_tensor,
 * read_exact, zero_fill, seal) with its contract in prose (src/weight_loader.rs:9-32,
 * AGENTS.md:55-67): parse config.json, the safetensors index and every shard header
 * first; reject duplicate, missing, unexpected, wrong-dtype, wrong-shape, overlapping
 * or out-of-range tensors before any CUDA-visible memory is touched; then fill the
 * final device storage from byte ranges of the files through a pinned staging ring
 * (cudaHostAlloc ring, pread, cudaMemcpyAsync, events), with one synchronisation
 * point at the end ("seal"). This section is that loader for the tensors of one MoE
 * layer, producing the layouts qs3_moe_layer_execute consumes.
 *
 * File formats: safetensors (8-byte little-endian header length, JSON header
 * {name: {dtype, shape, data_offsets}}, raw little-endian data) and the
 * model.safetensors.index.json / config.json files that accompany it. */

typedef struct qs3_checkpoint qs3_checkpoint;

/* Opens `directory`: with model.safetensors.index.json present its weight_map names the
 * shards, otherwise every *.safetensors file of the directory is a shard. Every shard
 * header is parsed and checked (header length inside the file, well-formed JSON, no
 * tensor name twice in a shard or across shards, known dtype, product(shape) * element
 * size == length of the byte range, ranges inside the file and pairwise disjoint; with
 * an index: every indexed tensor present in the shard it names and no tensor of a shard
 * missing from the index). Makes no CUDA call. */
qsfi_status qs3_checkpoint_open(qsfi_context* ctx, const char* directory, qs3_checkpoint** out);
void qs3_checkpoint_close(qs3_checkpoint* checkpoint); /* NULL is legal */
uint64_t qs3_checkpoint_num_tensors(const qs3_checkpoint* checkpoint);

#define QS3_CHECKPOINT_MAX_RANK 8u
typedef struct {
    const char* name;       /* owned by the checkpoint object */
    const char* file;       /* path of the shard, owned by the checkpoint object */
    const char* dtype_name; /* safetensors spelling: "BF16", "F8_E4M3", "U8", "F32", ... */
    qsfi_dtype dtype;       /* QSFI_DTYPE_INVALID for types qsfi_dtype cannot name (I64, F64, BOOL, ...) */
    uint32_t element_bytes;
    uint32_t rank;
    int64_t shape[QS3_CHECKPOINT_MAX_RANK];
    uint64_t file_offset; /* absolute offset of the first byte inside the shard */
    uint64_t bytes;
} qs3_checkpoint_tensor_info;
/* Tensors are numbered in name order. */
qsfi_status qs3_checkpoint_tensor_at(
    qsfi_context* ctx, const qs3_checkpoint* checkpoint, uint64_t index, qs3_checkpoint_tensor_info* out
);
qsfi_status qs3_checkpoint_find(
    qsfi_context* ctx, const qs3_checkpoint* checkpoint, const char* name, qs3_checkpoint_tensor_info* out
);
/* Copies the bytes of one tensor into host memory (dst_bytes must equal its size). */
qsfi_status qs3_checkpoint_read_host(
    qsfi_context* ctx, const qs3_checkpoint* checkpoint, const char* name, void* dst, uint64_t dst_bytes
);

/* MoE hyper-parameters of config.json (keys as Hugging Face's Qwen MoE configurations spell
 * them, read from the top level or from "text_config"): hidden_size, moe_intermediate_size,
 * num_experts, num_experts_per_tok, shared_expert_intermediate_size (0 when absent),
 * num_hidden_layers, norm_topk_prob (1 when absent), rms_norm_eps (1e-6 when absent). */
typedef struct {
    uint32_t hidden_size;
    uint32_t intermediate_size;
    uint32_t num_experts;
    uint32_t top_k;
    uint32_t shared_intermediate_size;
    uint32_t num_layers;
    uint32_t renormalize;
    float rms_norm_eps;
} qs3_checkpoint_moe_config;
qsfi_status qs3_checkpoint_read_moe_config(
    qsfi_context* ctx, const qs3_checkpoint* checkpoint, qs3_checkpoint_moe_config* out
);

/* How the routed experts are stored (AGENTS.md:45-47): BF16 checkpoints hold the fused
 * tensors <prefix>experts.gate_up_proj and <prefix>experts.down_proj; NVFP4 checkpoints
 * hold per expert e and per projection p in {gate_proj, up_proj, down_proj}
 *   <prefix>experts.<e>.<p>.weight          U8      [rows, k / 2]  two e2m1 codes per byte, low nibble = even k
 *   <prefix>experts.<e>.<p>.weight_scale    F8_E4M3 [rows, k / 16] one scale per 16 elements along k
 *   <prefix>experts.<e>.<p>.weight_scale_2  F32     [] or [1]      global scale of the matrix
 *   <prefix>experts.<e>.<p>.input_scale     F32     [] or [1]      global scale of the activations it multiplies
 * with value = e2m1 * weight_scale * weight_scale_2. The other tensors of the layer:
 *   <prefix>gate.weight                      BF16 [num_experts, hidden]   router
 *   <prefix>shared_expert.{gate,up,down}_proj.weight  (BF16, or NVFP4 with the four tensors above)
 *   <prefix>shared_expert_gate.weight        BF16 [1, hidden]
 * The fused BF16 expert tensors are accepted as [E, 2I, H] / [E, H, I] (the layout the
 * kernels read) or transposed, [E, H, 2I] / [E, I, H]; when hidden == 2 * intermediate the
 * two readings of gate_up_proj coincide and `fused_transposed` decides. */
typedef enum {
    QS3_CHECKPOINT_EXPERTS_BF16_FUSED = 0,
    QS3_CHECKPOINT_EXPERTS_NVFP4_SPLIT = 1
} qs3_checkpoint_expert_format;

typedef struct {
    const char* layer_prefix; /* e.g. "model.language_model.layers.3.mlp." */
    uint32_t hidden_size;
    uint32_t intermediate_size;
    uint32_t num_experts;
    uint32_t shared_intermediate_size; /* 0: the layer has no shared expert */
    uint32_t local_expert_offset;      /* first PHYSICAL expert position this rank holds */
    uint32_t local_num_experts;
    const uint32_t* expert_order;      /* optional [num_experts]: checkpoint expert id at each physical
                                          position (a placement that spreads hot experts over ranks);
                                          router rows are permuted the same way. NULL: identity */
    qs3_checkpoint_expert_format format;
    qsfi_moe_backend backend;          /* layout to produce: one of the two BF16 backends, or
                                          QSFI_MOE_BACKEND_FLASHINFER_NVFP4 (a BF16 checkpoint is
                                          then quantised on the device) */
    uint32_t fused_transposed;         /* BF16_FUSED, ambiguous shapes only: 1 = [E, H, 2I] / [E, I, H] */
} qs3_moe_layer_load_desc;

/* Device tensors of one loaded layer, ready to be copied into qs3_moe_layer_desc. They
 * all live inside the caller's device block. */
typedef struct {
    qsfi_tensor2 router_weight;               /* bf16 [num_experts, hidden], rows in physical order */
    qsfi_tensor3 gate_up_weight;              /* bf16 [E_local, 2I, H] or u8 [E_local, 2I, H/2] */
    qsfi_tensor1 gate_up_scale_tiled;         /* NVFP4 */
    qsfi_tensor1 gate_up_global_scale;        /* NVFP4 checkpoint: f32 [2 * E_local] (gate rows, up rows);
                                                 quantised here from BF16: f32 [E_local] */
    qsfi_tensor3 down_weight;
    qsfi_tensor1 down_scale_tiled;
    qsfi_tensor1 down_global_scale;           /* NVFP4: f32 [E_local] */
    qsfi_tensor3 shared_gate_up_weight;       /* data == NULL without a shared expert */
    qsfi_tensor1 shared_gate_up_scale_tiled;
    qsfi_tensor1 shared_gate_up_global_scale; /* f32 [2] from an NVFP4 checkpoint, f32 [1] otherwise */
    qsfi_tensor3 shared_down_weight;
    qsfi_tensor1 shared_down_scale_tiled;
    qsfi_tensor1 shared_down_global_scale;
    qsfi_tensor2 shared_gate_weight;          /* bf16 [1, hidden] */
    float act_global_scale;  /* NVFP4 checkpoints: max input_scale of all gate_proj / up_proj (every
                                expert of the layer, so that all ranks quantise tokens alike); else 1 */
    float act2_global_scale; /* max input_scale of all down_proj; else 1 */
} qs3_moe_layer_weights;

/* Validates the layer against the checkpoint (every expected tensor present with the
 * expected dtype and shape; no other tensor under layer_prefix) and returns the sizes of
 * the two device buffers qs3_checkpoint_load_moe_layer needs: `weight_bytes` for the
 * loaded tensors (kept) and `scratch_bytes` for load-time staging (may be freed after the
 * load). Makes no CUDA call. */
qsfi_status qs3_checkpoint_moe_layer_bytes(
    qsfi_context* ctx, const qs3_checkpoint* checkpoint, const qs3_moe_layer_load_desc* desc,
    size_t* weight_bytes, size_t* scratch_bytes
);

/* Loads the layer into `weights` (256-byte aligned device block of >= weight_bytes): file
 * byte ranges go through a ring of pinned host buffers and cudaMemcpyAsync on a copy stream
 * of the loader; scale re-tiling, transposes and quantisation then run on the context's
 * stream. Returns after the copy stream has drained and the device work is enqueued (work
 * on the context's stream is ordered after the copies); `scratch` may be released once the
 * context's stream has passed this point. */
qsfi_status qs3_checkpoint_load_moe_layer(
    qsfi_context* ctx, const qs3_checkpoint* checkpoint, const qs3_moe_layer_load_desc* desc,
    void* weights, size_t weight_bytes, void* scratch, size_t scratch_bytes, qs3_moe_layer_weights* out
);

#ifdef __cplusplus
}
#endif

#endif /* QS3_MOE_H */
