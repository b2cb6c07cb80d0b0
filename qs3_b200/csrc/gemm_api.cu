// qscb_* entry points: the dense bf16 projection lane that the MoE layer uses for
// the router logits and the shared expert (upstream qscb.h / qscb.cu), served by
// the tcgen05 kernel in gemm.cu instead of cuBLASLt.
#include "common.cuh"

#include <new>

struct qscb_context {
    int32_t device_ordinal;
    cudaStream_t stream;
    qsfi_error_info last_error;
};

namespace {

qsfi_status fail(qscb_context* ctx, qsfi_status status, qsfi_error_source source, int32_t code,
                 const char* fmt, ...)
{
    if (ctx == nullptr)
        return status;
    ctx->last_error.status = status;
    ctx->last_error.source = source;
    ctx->last_error.native_code = code;
    va_list args;
    va_start(args, fmt);
    std::vsnprintf(ctx->last_error.message, QSFI_ERROR_MESSAGE_BYTES, fmt, args);
    va_end(args);
    return status;
}

qsfi_status invalid(qscb_context* ctx, const char* msg)
{
    return fail(ctx, QSFI_STATUS_INVALID_ARGUMENT, QSFI_ERROR_SOURCE_QSFI, 0, "%s", msg);
}

} // namespace

extern "C" {

qsfi_status qscb_context_create(const qscb_context_desc* desc, qscb_context** out)
{
    if (out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    *out = nullptr;
    qscb_context* ctx = new (std::nothrow) qscb_context {};
    if (ctx == nullptr)
        return QSFI_STATUS_OUT_OF_MEMORY;
    ctx->device_ordinal = desc != nullptr ? desc->device_ordinal : -1;
    ctx->stream = desc != nullptr ? static_cast<cudaStream_t>(desc->stream) : nullptr;
    qs3::clear_error(&ctx->last_error);
    if (ctx->device_ordinal < 0) {
        // upstream binds to the device that is current at create time (qscb.h:30)
        if (cudaGetDevice(&ctx->device_ordinal) != cudaSuccess) {
            delete ctx;
            return QSFI_STATUS_CUDA_ERROR;
        }
    } else if (cudaSetDevice(ctx->device_ordinal) != cudaSuccess) {
        delete ctx;
        return QSFI_STATUS_CUDA_ERROR;
    }
    *out = ctx;
    return QSFI_STATUS_OK;
}

void qscb_context_destroy(qscb_context* ctx)
{
    delete ctx;
}

qsfi_status qscb_context_get_last_error(const qscb_context* ctx, qsfi_error_info* out)
{
    if (ctx == nullptr || out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    *out = ctx->last_error;
    return QSFI_STATUS_OK;
}

void qscb_context_clear_last_error(qscb_context* ctx)
{
    if (ctx != nullptr)
        qs3::clear_error(&ctx->last_error);
}

// out[rows, out_features] = alpha * x[rows, in] * weight[out, in]^T + beta * out,
// f32 accumulation, bf16 or f32 output, padded row strides accepted
// (upstream qscb.h:14-25, validation qscb.cu:160-262).
qsfi_status qscb_gemm_bf16(qscb_context* ctx, const qscb_bf16_gemm_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qs3::clear_error(&ctx->last_error);
    if (d == nullptr)
        return invalid(ctx, "desc is null");
    if (d->rows == 0 || d->in_features == 0 || d->out_features == 0)
        return invalid(ctx, "qscb GEMM dimensions must be non-zero");
    if (d->x.data == nullptr || d->weight.data == nullptr || d->out.data == nullptr)
        return invalid(ctx, "qscb GEMM tensors must not be null");
    if (d->x.dtype != QSFI_DTYPE_BF16 || d->weight.dtype != QSFI_DTYPE_BF16)
        return invalid(ctx, "qscb GEMM inputs must be bf16");
    if (d->out.dtype != QSFI_DTYPE_BF16 && d->out.dtype != QSFI_DTYPE_F32)
        return invalid(ctx, "qscb GEMM output must be bf16 or f32");
    if (d->x.stride[1] != 1 || d->weight.stride[1] != 1 || d->out.stride[1] != 1)
        return invalid(ctx, "qscb GEMM tensors must have unit inner stride");
    if (d->x.shape[0] != d->rows || d->x.shape[1] != d->in_features
        || d->weight.shape[0] != d->out_features || d->weight.shape[1] != d->in_features
        || d->out.shape[0] != d->rows || d->out.shape[1] != d->out_features)
        return invalid(ctx, "qscb GEMM tensor shape mismatch");
    if (d->x.stride[0] < d->in_features || d->weight.stride[0] < d->in_features
        || d->out.stride[0] < d->out_features)
        return invalid(ctx, "qscb GEMM row strides are smaller than the row length");
    if (cudaSetDevice(ctx->device_ordinal) != cudaSuccess)
        return fail(ctx, QSFI_STATUS_CUDA_ERROR, QSFI_ERROR_SOURCE_CUDA, 0, "cudaSetDevice failed");

    qs3::GemmProblem g {};
    g.a = d->x.data;
    g.a_rows = d->rows;
    g.a_pitch_bytes = static_cast<uint64_t>(d->x.stride[0]) * 2;
    g.b = d->weight.data;
    g.b_pitch_bytes = static_cast<uint64_t>(d->weight.stride[0]) * 2;
    g.groups = 1;
    g.n = d->out_features;
    g.k = d->in_features;
    g.epilogue = d->out.dtype == QSFI_DTYPE_F32 ? qs3::EPI_STORE_F32 : qs3::EPI_STORE_BF16;
    g.out = d->out.data;
    g.out_pitch_elems = static_cast<uint64_t>(d->out.stride[0]);
    g.alpha = d->alpha;
    g.beta = d->beta;
    const char* why = nullptr;
    cudaError_t err = qs3::launch_gemm(g, ctx->stream, &why);
    if (err == cudaSuccess)
        return QSFI_STATUS_OK;
    if (err == cudaErrorNotSupported)
        return fail(ctx, QSFI_STATUS_UNSUPPORTED, QSFI_ERROR_SOURCE_QSFI, 0, "qscb_gemm_bf16: %s",
                    why != nullptr ? why : "unsupported shape");
    return fail(ctx, qs3::status_from_cuda(err), QSFI_ERROR_SOURCE_CUDA, static_cast<int32_t>(err),
                "qscb_gemm_bf16: %s", cudaGetErrorString(err));
}

} // extern "C"
