// RMSNorm and fused add + RMSNorm: the two HBM-bound passes that bracket the MoE block in a
// transformer layer (upstream qsfi_rmsnorm / qsfi_fused_add_rmsnorm, qsfi_norm_rope.cu:89-206,
// 395-465, there a FlashInfer call), plus a variant that also emits the NVFP4 quantisation
// of the normalised tokens, which is what the MoE layer call consumes.
//
//   residual <- x + residual                      (stored in the tensor's dtype)
//   x        <- residual * rsqrt(mean(residual^2) + eps) * weight      (in place)
//
// One block per row; a thread keeps its elements in registers between the sum-of-squares
// pass and the scaling pass (rows up to 8192 elements for bf16, 4096 for f32; longer rows
// are re-read). Sums are taken in f32 from the unrounded x + residual, as upstream's checker
// does (tests_cuda_flashinfer_norm_rope.inc:190-217).
#include "common.cuh"
#include "nvfp4.cuh"

#include <cmath>
#include <limits>

namespace qs3 {

namespace {

constexpr int kNormThreads = 256;
constexpr int kNormCache = 4; // 16-byte vectors a thread keeps in registers

template <typename T> struct Vec;
template <> struct Vec<__nv_bfloat16> {
    static constexpr int kElems = 8;
    static __device__ __forceinline__ void unpack(const uint4& v, float* f)
    {
        const uint32_t w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            f[2 * j] = bf16_bits_to_f32(w[j] & 0xffffu);
            f[2 * j + 1] = bf16_bits_to_f32(w[j] >> 16);
        }
    }
    static __device__ __forceinline__ uint4 pack(const float* f)
    {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 r = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t*>(&r);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
};
template <> struct Vec<float> {
    static constexpr int kElems = 4;
    static __device__ __forceinline__ void unpack(const uint4& v, float* f)
    {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    static __device__ __forceinline__ uint4 pack(const float* f)
    {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                          __float_as_uint(f[3]));
    }
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};

struct NormParams {
    const void* x;        // input rows
    void* out;            // normalised rows (may alias x)
    void* residual;       // FUSED: read and updated
    const void* weight;
    uint32_t rows, hidden;
    uint64_t x_stride, out_stride, res_stride; // elements
    float eps, weight_bias;
    // optional NVFP4 copy of the bf16 output rows (token order, tiled scales)
    uint8_t* packed;
    uint8_t* scale_tiled;
    float global_scale;
};

__device__ __forceinline__ float block_sum(float v, float* s_part)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0)
        s_part[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) // fixed order: the same sum in every thread
        total += s_part[w];
    return total;
}

// VEC: rows are 16-byte aligned and hidden is a multiple of the vector width.
template <typename T, bool FUSED, bool VEC, bool QUANT>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(NormParams p)
{
    __shared__ float s_part[kNormThreads / 32];
    constexpr int E = Vec<T>::kElems;
    const uint32_t row = blockIdx.x;
    const T* x = static_cast<const T*>(p.x) + static_cast<uint64_t>(row) * p.x_stride;
    T* out = static_cast<T*>(p.out) + static_cast<uint64_t>(row) * p.out_stride;
    T* res = FUSED ? static_cast<T*>(p.residual) + static_cast<uint64_t>(row) * p.res_stride : nullptr;
    const T* w = static_cast<const T*>(p.weight);
    float sum_sq = 0.0f;

    if constexpr (VEC) {
        const uint32_t vecs = p.hidden / E;
        float cache[kNormCache][E];
#pragma unroll
        for (int c = 0; c < kNormCache; ++c) {
            const uint32_t i = threadIdx.x + c * kNormThreads;
            if (i < vecs) {
                Vec<T>::unpack(reinterpret_cast<const uint4*>(x)[i], cache[c]);
                if (FUSED) {
                    float r[E];
                    Vec<T>::unpack(reinterpret_cast<const uint4*>(res)[i], r);
#pragma unroll
                    for (int j = 0; j < E; ++j)
                        cache[c][j] += r[j];
                    reinterpret_cast<uint4*>(res)[i] = Vec<T>::pack(cache[c]);
                }
#pragma unroll
                for (int j = 0; j < E; ++j)
                    sum_sq += cache[c][j] * cache[c][j];
            }
        }
        for (uint32_t i = threadIdx.x + kNormCache * kNormThreads; i < vecs; i += kNormThreads) {
            float v[E];
            Vec<T>::unpack(reinterpret_cast<const uint4*>(x)[i], v);
            if (FUSED) {
                float r[E];
                Vec<T>::unpack(reinterpret_cast<const uint4*>(res)[i], r);
#pragma unroll
                for (int j = 0; j < E; ++j)
                    v[j] += r[j];
                reinterpret_cast<uint4*>(res)[i] = Vec<T>::pack(v);
            }
#pragma unroll
            for (int j = 0; j < E; ++j)
                sum_sq += v[j] * v[j];
        }
        const float total = block_sum(sum_sq, s_part);
        const float inv_rms = 1.0f / sqrtf(total / static_cast<float>(p.hidden) + p.eps);
#pragma unroll
        for (int c = 0; c < kNormCache; ++c) {
            const uint32_t i = threadIdx.x + c * kNormThreads;
            const uint32_t pair_mask = __ballot_sync(0xffffffffu, i < vecs); // lanes that quantise together
            (void)pair_mask;
            if (i < vecs) {
                float wv[E], y[E];
                Vec<T>::unpack(reinterpret_cast<const uint4*>(w)[i], wv);
#pragma unroll
                for (int j = 0; j < E; ++j)
                    y[j] = cache[c][j] * inv_rms * (p.weight_bias + wv[j]);
                const uint4 packed_row = Vec<T>::pack(y);
                reinterpret_cast<uint4*>(out)[i] = packed_row;
                if constexpr (QUANT) {
                    // two threads hold one 16-element block: exchange halves, the even one writes
                    float blk[16];
                    Vec<T>::unpack(packed_row, y); // quantise what was stored (bf16-rounded)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float other = __shfl_xor_sync(pair_mask, y[j], 1);
                        blk[j] = (threadIdx.x & 1) ? other : y[j];
                        blk[8 + j] = (threadIdx.x & 1) ? y[j] : other;
                    }
                    uint32_t lo, hi;
                    const uint8_t code = quantize_block16(blk, p.global_scale, &lo, &hi);
                    if ((threadIdx.x & 1) == 0) {
                        const uint32_t kb = i / 2; // 16-element block index along the row
                        *reinterpret_cast<uint2*>(p.packed + static_cast<uint64_t>(row) * (p.hidden / 2) + kb * 8)
                            = make_uint2(lo, hi);
                        p.scale_tiled[tiled_scale_offset(row, kb, p.hidden / 64)] = code;
                    }
                }
            }
        }
        for (uint32_t i = threadIdx.x + kNormCache * kNormThreads; i < vecs; i += kNormThreads) {
            float v[E], wv[E];
            Vec<T>::unpack(reinterpret_cast<const uint4*>(FUSED ? res : x)[i], v); // long rows: re-read
            Vec<T>::unpack(reinterpret_cast<const uint4*>(w)[i], wv);
#pragma unroll
            for (int j = 0; j < E; ++j)
                v[j] = v[j] * inv_rms * (p.weight_bias + wv[j]);
            reinterpret_cast<uint4*>(out)[i] = Vec<T>::pack(v);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < p.hidden; i += kNormThreads) {
            float v = Vec<T>::load(x + i);
            if (FUSED) {
                v += Vec<T>::load(res + i);
                Vec<T>::store(res + i, v);
            }
            sum_sq += v * v;
        }
        const float total = block_sum(sum_sq, s_part);
        const float inv_rms = 1.0f / sqrtf(total / static_cast<float>(p.hidden) + p.eps);
        // in the fused form x aliases out, so the second pass takes the sum from the residual
        // row it was stored to (rounded to the tensor's dtype)
        for (uint32_t i = threadIdx.x; i < p.hidden; i += kNormThreads) {
            const float v = FUSED ? Vec<T>::load(res + i) : Vec<T>::load(x + i);
            Vec<T>::store(out + i, v * inv_rms * (p.weight_bias + Vec<T>::load(w + i)));
        }
    }
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

template <typename T, bool FUSED> cudaError_t launch_norm(const NormParams& p, bool quant, cudaStream_t stream)
{
    constexpr uint64_t E = Vec<T>::kElems;
    const bool vec = p.hidden % E == 0 && aligned16(p.x) && aligned16(p.out) && aligned16(p.weight)
        && p.x_stride % E == 0 && p.out_stride % E == 0
        && (!FUSED || (aligned16(p.residual) && p.res_stride % E == 0));
    if (p.rows == 0)
        return cudaSuccess;
    if (quant) {
        if constexpr (sizeof(T) == 2 && FUSED) {
            if (!vec)
                return cudaErrorInvalidValue;
            rmsnorm_kernel<T, true, true, true><<<p.rows, kNormThreads, 0, stream>>>(p);
        } else {
            return cudaErrorInvalidValue;
        }
    } else if (vec) {
        rmsnorm_kernel<T, FUSED, true, false><<<p.rows, kNormThreads, 0, stream>>>(p);
    } else {
        rmsnorm_kernel<T, FUSED, false, false><<<p.rows, kNormThreads, 0, stream>>>(p);
    }
    note_launch();
    return cudaGetLastError();
}

// ---- validation, same checks and messages as upstream qsfi_norm_rope.cu:72-146, 208-238 ----

bool supported_float_dtype(qsfi_dtype dtype) { return dtype == QSFI_DTYPE_BF16 || dtype == QSFI_DTYPE_F32; }

const char* dtype_name(qsfi_dtype dtype)
{
    return dtype == QSFI_DTYPE_F32 ? "f32" : dtype == QSFI_DTYPE_BF16 ? "bf16" : "unsupported";
}

template <typename Tensor>
qsfi_status check_tensor(qsfi_context* ctx, const Tensor& t, const char* name, qsfi_dtype dtype)
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

bool row_major_inner(const qsfi_tensor2& t) { return t.stride[1] == 1 && t.stride[0] >= t.shape[1]; }

qsfi_status require_u32(qsfi_context* ctx, int64_t value, const char* name)
{
    if (value < 0 || static_cast<uint64_t>(value) > std::numeric_limits<uint32_t>::max())
        return set_invalid_arg(ctx, "%s must fit in uint32_t", name);
    return QSFI_STATUS_OK;
}

qsfi_status validate_common(qsfi_context* ctx, const qsfi_tensor2& x, const qsfi_tensor1& weight,
                            const qsfi_tensor2& out, uint32_t hidden_size, float eps, const char* op)
{
    if (hidden_size == 0)
        return set_invalid_arg(ctx, "%s hidden_size must be non-zero", op);
    if (!supported_float_dtype(x.dtype))
        return set_unsupported(ctx, "%s supports only bf16/f32 tensors, got %s", op, dtype_name(x.dtype));
    qsfi_status status = check_tensor(ctx, x, "x", x.dtype);
    if (status != QSFI_STATUS_OK)
        return status;
    status = check_tensor(ctx, weight, "weight", x.dtype);
    if (status != QSFI_STATUS_OK)
        return status;
    status = check_tensor(ctx, out, "out", x.dtype);
    if (status != QSFI_STATUS_OK)
        return status;
    if (x.shape[1] != static_cast<int64_t>(hidden_size) || out.shape[1] != x.shape[1]
        || weight.shape[0] != x.shape[1])
        return set_invalid_arg(ctx, "%s tensors must use hidden_size as their innermost extent", op);
    if (out.shape[0] != x.shape[0])
        return set_invalid_arg(ctx, "%s out row count must match x", op);
    if (!row_major_inner(x) || !row_major_inner(out) || weight.stride[0] != 1)
        return set_invalid_arg(ctx, "%s requires contiguous hidden dimension and contiguous weight", op);
    status = require_u32(ctx, x.shape[0], "x.shape[0]");
    if (status != QSFI_STATUS_OK)
        return status;
    status = require_u32(ctx, x.stride[0], "x.stride[0]");
    if (status != QSFI_STATUS_OK)
        return status;
    status = require_u32(ctx, out.stride[0], "out.stride[0]");
    if (status != QSFI_STATUS_OK)
        return status;
    if (!std::isfinite(eps) || eps <= 0.0f)
        return set_invalid_arg(ctx, "rmsnorm eps must be finite and > 0");
    return QSFI_STATUS_OK;
}

qsfi_status validate_fused(qsfi_context* ctx, const qsfi_fused_add_rmsnorm_desc* d)
{
    qsfi_status status = validate_common(ctx, d->x, d->weight, d->out, d->hidden_size, d->eps, "fused_add_rmsnorm");
    if (status != QSFI_STATUS_OK)
        return status;
    status = check_tensor(ctx, d->residual_inout, "residual_inout", d->x.dtype);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d->x.shape[0] != d->residual_inout.shape[0] || d->x.shape[1] != d->residual_inout.shape[1])
        return set_invalid_arg(ctx, "fused_add_rmsnorm residual_inout shape must match x");
    if (!row_major_inner(d->residual_inout))
        return set_invalid_arg(ctx, "fused_add_rmsnorm residual_inout hidden dimension must be contiguous");
    if (d->out.data != d->x.data || d->out.shape[0] != d->x.shape[0] || d->out.shape[1] != d->x.shape[1]
        || d->out.stride[0] != d->x.stride[0] || d->out.stride[1] != d->x.stride[1])
        return set_invalid_arg(ctx, "fused_add_rmsnorm out must alias x exactly");
    return require_u32(ctx, d->residual_inout.stride[0], "residual_inout.stride[0]");
}

NormParams fused_params(const qsfi_fused_add_rmsnorm_desc* d)
{
    NormParams p {};
    p.x = d->x.data;
    p.out = d->x.data;
    p.residual = d->residual_inout.data;
    p.weight = d->weight.data;
    p.rows = static_cast<uint32_t>(d->x.shape[0]);
    p.hidden = d->hidden_size;
    p.x_stride = p.out_stride = static_cast<uint64_t>(d->x.stride[0]);
    p.res_stride = static_cast<uint64_t>(d->residual_inout.stride[0]);
    p.eps = d->eps;
    return p;
}

} // namespace
} // namespace qs3

using namespace qs3;

extern "C" {

qsfi_status qsfi_rmsnorm(qsfi_context* ctx, const qsfi_rmsnorm_desc* desc)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    if (desc == nullptr)
        return set_invalid_arg(ctx, "rmsnorm desc must not be null");
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_common(ctx, desc->x, desc->weight, desc->out, desc->hidden_size, desc->eps, "rmsnorm");
    if (status != QSFI_STATUS_OK)
        return status;
    if (!std::isfinite(desc->weight_bias))
        return set_invalid_arg(ctx, "rmsnorm weight_bias must be finite");
    if (desc->weight_bias != 0.0f && desc->weight_bias != 1.0f)
        return set_unsupported(ctx, "rmsnorm weight_bias must be 0.0 or 1.0");
    NormParams p {};
    p.x = desc->x.data;
    p.out = desc->out.data;
    p.weight = desc->weight.data;
    p.rows = static_cast<uint32_t>(desc->x.shape[0]);
    p.hidden = desc->hidden_size;
    p.x_stride = static_cast<uint64_t>(desc->x.stride[0]);
    p.out_stride = static_cast<uint64_t>(desc->out.stride[0]);
    p.eps = desc->eps;
    p.weight_bias = desc->weight_bias;
    const cudaError_t err = desc->x.dtype == QSFI_DTYPE_BF16
        ? launch_norm<__nv_bfloat16, false>(p, false, ctx->stream)
        : launch_norm<float, false>(p, false, ctx->stream);
    return set_cuda_error(ctx, err, "rmsnorm");
}

qsfi_status qsfi_fused_add_rmsnorm(qsfi_context* ctx, const qsfi_fused_add_rmsnorm_desc* desc)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    if (desc == nullptr)
        return set_invalid_arg(ctx, "fused_add_rmsnorm desc must not be null");
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_fused(ctx, desc);
    if (status != QSFI_STATUS_OK)
        return status;
    const NormParams p = fused_params(desc);
    const cudaError_t err = desc->x.dtype == QSFI_DTYPE_BF16
        ? launch_norm<__nv_bfloat16, true>(p, false, ctx->stream)
        : launch_norm<float, true>(p, false, ctx->stream);
    return set_cuda_error(ctx, err, "fused_add_rmsnorm");
}

qsfi_status qs3_fused_add_rmsnorm_nvfp4(qsfi_context* ctx, const qs3_fused_add_rmsnorm_nvfp4_desc* desc)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    if (desc == nullptr)
        return set_invalid_arg(ctx, "fused_add_rmsnorm desc must not be null");
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    status = validate_fused(ctx, &desc->norm);
    if (status != QSFI_STATUS_OK)
        return status;
    const uint32_t hidden = desc->norm.hidden_size;
    const int64_t rows = desc->norm.x.shape[0];
    if (desc->norm.x.dtype != QSFI_DTYPE_BF16)
        return set_unsupported(ctx, "fused_add_rmsnorm with NVFP4 output supports only bf16 tensors");
    if (hidden % 64 != 0 || hidden > 8192)
        return set_unsupported(ctx, "fused_add_rmsnorm with NVFP4 output needs hidden_size divisible by 64 and <= 8192");
    if (desc->packed.data == nullptr || desc->packed.dtype != QSFI_DTYPE_U8 || desc->packed.shape[0] < rows
        || desc->packed.shape[1] != hidden / 2 || !contiguous2(desc->packed))
        return set_invalid_arg(ctx, "packed must be a contiguous u8 [rows, hidden_size/2] tensor");
    if (desc->scale_tiled.data == nullptr
        || static_cast<uint64_t>(desc->scale_tiled.shape[0])
            < qs3_nvfp4_tiled_scale_bytes(static_cast<uint64_t>(rows), hidden))
        return set_invalid_arg(ctx, "scale_tiled is too small for [rows, hidden_size]");
    if (!std::isfinite(desc->global_scale) || desc->global_scale < 0.0f)
        return set_invalid_arg(ctx, "global_scale must be finite and >= 0");
    NormParams p = fused_params(&desc->norm);
    p.packed = static_cast<uint8_t*>(desc->packed.data);
    p.scale_tiled = static_cast<uint8_t*>(desc->scale_tiled.data);
    p.global_scale = desc->global_scale == 0.0f ? 1.0f : desc->global_scale;
    const cudaError_t err = launch_norm<__nv_bfloat16, true>(p, true, ctx->stream);
    if (err == cudaErrorInvalidValue)
        return set_invalid_arg(ctx, "fused_add_rmsnorm with NVFP4 output needs 16-byte aligned rows");
    return set_cuda_error(ctx, err, "qs3_fused_add_rmsnorm_nvfp4");
}

} // extern "C"
