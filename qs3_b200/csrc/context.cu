// Context life cycle, error record and build/target queries of the C ABI.
// Behaviour follows upstream qsfi_context.cu:10-283 for the entry points the
// MoE path uses; the build target answered here is sm_100 (compute 10.0).
#include "common.cuh"

#include <atomic>
#include <mutex>
#include <new>

namespace qs3 {

void clear_error(qsfi_error_info* err)
{
    if (err == nullptr)
        return;
    err->status = QSFI_STATUS_OK;
    err->source = QSFI_ERROR_SOURCE_NONE;
    err->native_code = 0;
    err->message[0] = '\0';
}

static qsfi_status record(qsfi_context* ctx, qsfi_status status, qsfi_error_source source,
                          int32_t native_code, const char* fmt, va_list args)
{
    if (ctx == nullptr)
        return status;
    qsfi_error_info& e = ctx->last_error;
    e.status = status;
    e.source = source;
    e.native_code = native_code;
    std::vsnprintf(e.message, QSFI_ERROR_MESSAGE_BYTES, fmt, args);
    e.message[QSFI_ERROR_MESSAGE_BYTES - 1] = '\0';
    return status;
}

qsfi_status set_error(qsfi_context* ctx, qsfi_status status, qsfi_error_source source,
                      int32_t native_code, const char* fmt, ...)
{
    va_list args;
    va_start(args, fmt);
    status = record(ctx, status, source, native_code, fmt, args);
    va_end(args);
    return status;
}

qsfi_status set_invalid_arg(qsfi_context* ctx, const char* fmt, ...)
{
    va_list args;
    va_start(args, fmt);
    qsfi_status s = record(ctx, QSFI_STATUS_INVALID_ARGUMENT, QSFI_ERROR_SOURCE_QSFI, 0, fmt, args);
    va_end(args);
    return s;
}

qsfi_status set_unsupported(qsfi_context* ctx, const char* fmt, ...)
{
    va_list args;
    va_start(args, fmt);
    qsfi_status s = record(ctx, QSFI_STATUS_UNSUPPORTED, QSFI_ERROR_SOURCE_QSFI, 0, fmt, args);
    va_end(args);
    return s;
}

qsfi_status status_from_cuda(cudaError_t err)
{
    if (err == cudaSuccess)
        return QSFI_STATUS_OK;
    return err == cudaErrorMemoryAllocation ? QSFI_STATUS_OUT_OF_MEMORY : QSFI_STATUS_CUDA_ERROR;
}

qsfi_status set_cuda_error(qsfi_context* ctx, cudaError_t err, const char* op)
{
    if (err == cudaSuccess)
        return QSFI_STATUS_OK;
    return set_error(ctx, status_from_cuda(err), QSFI_ERROR_SOURCE_CUDA, static_cast<int32_t>(err),
                     "%s: %s", op, cudaGetErrorString(err));
}

qsfi_status activate_context(qsfi_context* ctx)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    if (ctx->device_ordinal < 0)
        return QSFI_STATUS_OK;
    return set_cuda_error(ctx, cudaSetDevice(ctx->device_ordinal), "cudaSetDevice");
}

// One error word per device: a file-scope device variable, so no allocation is
// needed; its device address is looked up once per device.
__device__ uint32_t g_device_error_word = 0;

uint32_t* device_error_word()
{
    static std::mutex mu;
    static uint32_t* words[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (words[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_error_word) != cudaSuccess)
            return nullptr;
        words[dev] = static_cast<uint32_t*>(p);
    }
    return words[dev];
}

static std::atomic<uint64_t> g_launches { 0 };
void note_launch(uint32_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

struct StageRecorder {
    bool on = false;
    bool created = false;
    int count = 0;
    cudaEvent_t ev[64];
    int ids[64];
};
static StageRecorder g_rec;

bool stage_recording() { return g_rec.on; }

#if QSFI_ENABLE_CHECKED_VALIDATION
__device__ int g_checked_flag;

int* checked_flag_reset(cudaStream_t stream, cudaError_t* err)
{
    int* flag = nullptr;
    *err = cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), g_checked_flag);
    if (*err == cudaSuccess)
        *err = cudaMemsetAsync(flag, 0, sizeof(int), stream);
    return flag;
}

bool checked_flag_finish(cudaStream_t stream, cudaError_t* err)
{
    int* flag = nullptr;
    int host = 0;
    *err = cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), g_checked_flag);
    if (*err == cudaSuccess)
        *err = cudaMemcpyAsync(&host, flag, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (*err == cudaSuccess)
        *err = cudaStreamSynchronize(stream);
    return host != 0;
}
#endif

void stage_mark(cudaStream_t stream, int stage)
{
    if (!g_rec.on || g_rec.count >= 64)
        return;
    cudaEventRecord(g_rec.ev[g_rec.count], stream);
    g_rec.ids[g_rec.count++] = stage;
}

} // namespace qs3

using namespace qs3;

extern "C" {

const char* qsfi_status_string(qsfi_status status)
{
    static const char* const names[] = { "ok",         "invalid argument", "unsupported",
                                         "out of memory", "cuda error",    "backend error",
                                         "internal error" };
    const int i = static_cast<int>(status);
    return (i >= 0 && i <= 6) ? names[i] : "unknown status";
}

qsfi_status qsfi_context_create(const qsfi_context_desc* desc, qsfi_context** out)
{
    if (out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    *out = nullptr;
    qsfi_context* ctx = new (std::nothrow) qsfi_context {};
    if (ctx == nullptr)
        return QSFI_STATUS_OUT_OF_MEMORY;
    ctx->device_ordinal = desc != nullptr ? desc->device_ordinal : -1;
    ctx->stream = desc != nullptr ? static_cast<cudaStream_t>(desc->stream) : nullptr;
    clear_error(&ctx->last_error);
    if (ctx->device_ordinal >= 0 && cudaSetDevice(ctx->device_ordinal) != cudaSuccess) {
        delete ctx;
        return QSFI_STATUS_CUDA_ERROR;
    }
    *out = ctx;
    return QSFI_STATUS_OK;
}

void qsfi_context_destroy(qsfi_context* ctx)
{
    if (ctx == nullptr)
        return;
    if (ctx->float_workspace != nullptr) {
        if (ctx->device_ordinal >= 0)
            cudaSetDevice(ctx->device_ordinal);
        cudaFree(ctx->float_workspace);
    }
    delete ctx;
}

qsfi_status qsfi_context_set_stream(qsfi_context* ctx, qsfi_cuda_stream stream)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    ctx->stream = static_cast<cudaStream_t>(stream);
    clear_error(&ctx->last_error);
    return QSFI_STATUS_OK;
}

qsfi_status qsfi_get_build_config(qsfi_build_config* out)
{
    if (out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    out->target_sm = 100;
    out->target_compute_capability_major = 10;
    out->target_compute_capability_minor = 0;
    out->assume_fp8 = 1;
    out->assume_fp4 = 1;
    out->assume_pdl = 0;
    out->gemm_backend = 0;
    return QSFI_STATUS_OK;
}

qsfi_status qsfi_context_get_info(qsfi_context* ctx, qsfi_context_info* out)
{
    if (ctx == nullptr || out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    int device = ctx->device_ordinal;
    if (device < 0) {
        cudaError_t err = cudaGetDevice(&device);
        if (err != cudaSuccess)
            return set_cuda_error(ctx, err, "cudaGetDevice");
    }
    int major = 0, minor = 0;
    cudaError_t err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (err == cudaSuccess)
        err = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "cudaDeviceGetAttribute");
    out->runtime_compute_capability_major = static_cast<uint32_t>(major);
    out->runtime_compute_capability_minor = static_cast<uint32_t>(minor);
    return QSFI_STATUS_OK;
}

qsfi_status qsfi_context_validate_target(qsfi_context* ctx)
{
    qsfi_context_info info {};
    qsfi_status status = qsfi_context_get_info(ctx, &info);
    if (status != QSFI_STATUS_OK)
        return status;
    if (info.runtime_compute_capability_major != 10 || info.runtime_compute_capability_minor != 0) {
        return set_unsupported(
            ctx, "runtime compute capability %u.%u does not match qsfi build target %u.%u",
            info.runtime_compute_capability_major, info.runtime_compute_capability_minor, 10u, 0u);
    }
    return QSFI_STATUS_OK;
}

qsfi_status qsfi_context_get_last_error(const qsfi_context* ctx, qsfi_error_info* out)
{
    if (ctx == nullptr || out == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    *out = ctx->last_error;
    return QSFI_STATUS_OK;
}

void qsfi_context_clear_last_error(qsfi_context* ctx)
{
    if (ctx != nullptr)
        clear_error(&ctx->last_error);
}

qsfi_status qs3_moe_read_device_error(qsfi_context* ctx, uint32_t* code)
{
    if (ctx == nullptr || code == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    uint32_t* word = device_error_word();
    if (word == nullptr)
        return set_error(ctx, QSFI_STATUS_CUDA_ERROR, QSFI_ERROR_SOURCE_CUDA, 0,
                         "device error word unavailable");
    cudaError_t err = cudaStreamSynchronize(ctx->stream);
    if (err == cudaSuccess)
        err = cudaMemcpy(code, word, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (err == cudaSuccess && *code != 0)
        err = cudaMemset(word, 0, sizeof(uint32_t));
    return set_cuda_error(ctx, err, "qs3_moe_read_device_error");
}

uint64_t qs3_moe_launch_count(void)
{
    return g_launches.load(std::memory_order_relaxed);
}

qsfi_status qs3_moe_profile_begin(qsfi_context* ctx)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (!g_rec.created) {
        for (int i = 0; i < 64; ++i) {
            cudaError_t err = cudaEventCreate(&g_rec.ev[i]);
            if (err != cudaSuccess)
                return set_cuda_error(ctx, err, "cudaEventCreate");
        }
        g_rec.created = true;
    }
    g_rec.count = 0;
    g_rec.on = true;
    return QSFI_STATUS_OK;
}

qsfi_status qs3_moe_profile_end(qsfi_context* ctx, int32_t* stage_ids, float* stage_ms, uint32_t capacity,
                                uint32_t* count)
{
    if (ctx == nullptr || stage_ids == nullptr || stage_ms == nullptr || count == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    g_rec.on = false;
    *count = 0;
    cudaError_t err = cudaStreamSynchronize(ctx->stream);
    if (err != cudaSuccess)
        return set_cuda_error(ctx, err, "cudaStreamSynchronize");
    for (int i = 0; i + 1 < g_rec.count && *count < capacity; ++i) {
        if (g_rec.ids[i] == STAGE_END)
            continue;
        float ms = 0.0f;
        err = cudaEventElapsedTime(&ms, g_rec.ev[i], g_rec.ev[i + 1]);
        if (err != cudaSuccess)
            return set_cuda_error(ctx, err, "cudaEventElapsedTime");
        stage_ids[*count] = g_rec.ids[i];
        stage_ms[*count] = ms;
        *count += 1;
    }
    return QSFI_STATUS_OK;
}

} // extern "C"
