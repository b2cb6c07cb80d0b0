// Router top-k and the two element-wise helpers of the MoE layer
// (qscu_router_topk, qscu_silu_and_mul_bf16, qscu_qwen36_shared_expert_gate_add_bf16).
#include "common.cuh"

#include <climits>
#include <cmath>

namespace qs3 {

namespace {

constexpr uint32_t kRouterMaxTopK = 16;      // upstream qscu.cu:29
constexpr uint32_t kRouterMaxExperts = 4096; // upstream qscu.cu:30
constexpr float kRouterNegInf = -3.4028234663852886e38f; // upstream qscu.cu:31
constexpr int kRouterWarps = 4;

// Ordering of upstream better_router_candidate (qscu.cu:888-892) extended with
// "no candidate" (id == INT_MAX), which loses against every real candidate.
__device__ __forceinline__ bool candidate_better(float s1, int i1, float s2, int i2)
{
    if (i1 == INT_MAX)
        return false;
    if (i2 == INT_MAX)
        return true;
    return s1 > s2 || (s1 == s2 && i1 < i2);
}

// One warp per token. The token's select scores live in shared memory; each of
// the top_k rounds is a warp arg-max over the not-yet-taken experts, which yields
// exactly the list upstream's insertion loop builds (descending score, ties to
// the lower id, NaN and anything below -FLT_MAX never selected; qscu.cu:894-971).
template <typename LogitT>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const LogitT* __restrict__ logits, const float* __restrict__ bias,
                   int32_t* __restrict__ topk_ids, float* __restrict__ topk_weights,
                   uint32_t num_tokens, uint32_t num_experts, uint32_t top_k, int sigmoid_score,
                   int renormalize, float scaling)
{
    extern __shared__ float s_scores[];
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t token = blockIdx.x * kRouterWarps + warp;
    if (token >= num_tokens)
        return;
    float* sc = s_scores + static_cast<size_t>(warp) * num_experts;
    const LogitT* row = logits + static_cast<size_t>(token) * num_experts;

    // pass 1: stage logits (+ bias), running max
    float vmax = kRouterNegInf;
    for (uint32_t e = lane; e < num_experts; e += 32) {
        float l;
        if constexpr (sizeof(LogitT) == 2)
            l = __bfloat162float(row[e]);
        else
            l = row[e];
        if (bias != nullptr)
            l += bias[e];
        sc[e] = l;
        if (l > vmax)
            vmax = l;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, vmax, o);
        if (other > vmax)
            vmax = other;
    }
    __syncwarp();

    // pass 2: softmax denominator, or replace logits by sigmoid scores
    float denom = 0.0f;
    if (!sigmoid_score) {
        for (uint32_t e = lane; e < num_experts; e += 32)
            denom += expf(sc[e] - vmax);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            denom += __shfl_xor_sync(0xffffffffu, denom, o);
    } else {
        for (uint32_t e = lane; e < num_experts; e += 32)
            sc[e] = sigmoid_fast(sc[e]);
        __syncwarp();
    }

    // top_k rounds of warp arg-max
    float my_weight = 0.0f; // lane p keeps slot p
    int my_id = 0;
    for (uint32_t pos = 0; pos < top_k; ++pos) {
        float bs = kRouterNegInf;
        int bi = INT_MAX;
        for (uint32_t e = lane; e < num_experts; e += 32) {
            const float s = sc[e];
            // valid candidates are exactly the values upstream's insertion accepts
            if (s >= kRouterNegInf && candidate_better(s, static_cast<int>(e), bs, bi)) {
                bs = s;
                bi = static_cast<int>(e);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float os = __shfl_xor_sync(0xffffffffu, bs, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (candidate_better(os, oi, bs, bi)) {
                bs = os;
                bi = oi;
            }
        }
        float w = 0.0f;
        int id = static_cast<int>(pos); // unfilled slot: id = slot, weight 0 (qscu.cu:945-949)
        if (bi != INT_MAX) {
            id = bi;
            if (sigmoid_score)
                w = bs;
            else
                w = denom > 0.0f ? expf(bs - vmax) / denom : 0.0f;
            if ((static_cast<uint32_t>(bi) & 31u) == lane)
                sc[bi] = __int_as_float(0x7fc00000); // taken: NaN never qualifies again
        }
        __syncwarp();
        if (lane == pos) {
            my_weight = w;
            my_id = id;
        }
    }

    // renormalise: sum in slot order like upstream (qscu.cu:944-960)
    float sum = 0.0f;
    for (uint32_t pos = 0; pos < top_k; ++pos)
        sum += __shfl_sync(0xffffffffu, my_weight, pos);
    const float renorm = renormalize ? 1.0f / fmaxf(sum, 1.0e-20f) : 1.0f;
    if (lane < top_k) {
        topk_ids[static_cast<size_t>(token) * top_k + lane] = my_id;
        topk_weights[static_cast<size_t>(token) * top_k + lane] = my_weight * renorm * scaling;
    }
}

// Order-preserving map float -> u32 for the values upstream's insertion accepts
// (score >= -FLT_MAX, not NaN); everything else maps to 0 and never wins. -0 is folded
// into +0 so that equal floats give equal keys.
__device__ __forceinline__ uint32_t score_key(float s)
{
    if (!(s >= kRouterNegInf))
        return 0u;
    const uint32_t b = __float_as_uint(s + 0.0f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float key_score(uint32_t k)
{
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Same routing as router_topk_kernel for num_experts <= 32 * ITEMS, with the token's
// scores held in registers (lane owns experts lane, lane + 32, ...). A round is a
// register arg-max per lane, one redux.sync max over the keys and one redux.sync min
// over the candidate ids (ties go to the lowest id, as upstream's insertion does).
template <typename LogitT, int ITEMS>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_reg_kernel(const LogitT* __restrict__ logits, const float* __restrict__ bias,
                       int32_t* __restrict__ topk_ids, float* __restrict__ topk_weights,
                       uint32_t num_tokens, uint32_t num_experts, uint32_t top_k, int sigmoid_score,
                       int renormalize, float scaling)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t token = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
    if (token >= num_tokens)
        return;
    const LogitT* row = logits + static_cast<size_t>(token) * num_experts;

    float val[ITEMS];
    uint32_t key[ITEMS];
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
        const uint32_t e = lane + 32u * j;
        float l = __uint_as_float(0x7fc00000u); // padding: NaN, never selected, skipped below
        if (e < num_experts) {
            if constexpr (sizeof(LogitT) == 2)
                l = __bfloat162float(row[e]);
            else
                l = row[e];
            if (bias != nullptr)
                l += bias[e];
        }
        val[j] = l;
    }
    uint32_t kmax = 0;
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
        key[j] = score_key(val[j]);
        kmax = max(kmax, key[j]);
    }
    kmax = __reduce_max_sync(0xffffffffu, kmax);
    const float vmax = kmax != 0u ? key_score(kmax) : kRouterNegInf;

    float denom = 0.0f;
    if (!sigmoid_score) {
#pragma unroll
        for (int j = 0; j < ITEMS; ++j)
            if (lane + 32u * j < num_experts)
                denom += expf(val[j] - vmax);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            denom += __shfl_xor_sync(0xffffffffu, denom, o);
    } else {
#pragma unroll
        for (int j = 0; j < ITEMS; ++j)
            key[j] = lane + 32u * j < num_experts ? score_key(sigmoid_fast(val[j])) : 0u;
    }

    float my_weight = 0.0f;
    int my_id = 0;

    // Fast path. The arg-max rounds below cost ~3 * ITEMS integer instructions each, and the integer pipe,
    // not memory, bounds this kernel (ncu: 1800 instructions per token, ALU pipe 70 % busy). Most of that
    // work is spent on keys that cannot win: tau, the top_k-th largest of the 32 lane maxima, is a lower
    // bound of the top_k-th largest key (top_k different lanes hold a key >= tau), so every winner is
    // among the keys >= tau. Those are usually a dozen or two; they are compacted to one per lane and the
    // rounds run on them. Ties keep upstream's rule (equal keys: lowest id), because all keys equal to
    // the boundary value are candidates too. Falls back to the full rounds when fewer than top_k lanes
    // hold a valid key (tau == 0) or more than 32 keys reach tau.
    __shared__ uint32_t s_ck[kRouterWarps][32];
    __shared__ uint32_t s_cid[kRouterWarps][32];
    bool fast = top_k <= 32;
    uint32_t tau = 0;
    if (fast) {
        uint32_t t = 0;
#pragma unroll
        for (int j = 0; j < ITEMS; ++j)
            t = max(t, key[j]);
        for (uint32_t pos = 0; pos < top_k; ++pos) {
            tau = __reduce_max_sync(0xffffffffu, t);
            const uint32_t holders = __ballot_sync(0xffffffffu, t == tau);
            if (lane == static_cast<uint32_t>(__ffs(static_cast<int>(holders)) - 1))
                t = 0; // one lane per step, so that equal maxima count once each
        }
        fast = tau != 0u;
    }
    if (fast) {
        uint32_t cnt = 0;
#pragma unroll
        for (int j = 0; j < ITEMS; ++j)
            cnt += key[j] >= tau ? 1u : 0u;
        uint32_t incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= static_cast<uint32_t>(o))
                incl += v;
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        fast = total <= 32u;
        if (fast) {
            const uint32_t wslot = threadIdx.x >> 5;
            uint32_t at = incl - cnt;
#pragma unroll
            for (int j = 0; j < ITEMS; ++j)
                if (key[j] >= tau) {
                    s_ck[wslot][at] = key[j];
                    s_cid[wslot][at] = lane + 32u * static_cast<uint32_t>(j);
                    ++at;
                }
            __syncwarp();
            uint32_t ck = lane < total ? s_ck[wslot][lane] : 0u;
            const uint32_t cid = lane < total ? s_cid[wslot][lane] : 0xffffffffu;
            for (uint32_t pos = 0; pos < top_k; ++pos) {
                const uint32_t top = __reduce_max_sync(0xffffffffu, ck); // never 0: total >= top_k candidates
                const uint32_t win = __reduce_min_sync(0xffffffffu, ck == top ? cid : 0xffffffffu);
                const float sc = key_score(top);
                const float w = sigmoid_score ? sc : (denom > 0.0f ? expf(sc - vmax) / denom : 0.0f);
                if (cid == win)
                    ck = 0u;
                if (lane == pos) {
                    my_weight = w;
                    my_id = static_cast<int>(win);
                }
            }
        }
    }
    for (uint32_t pos = 0; !fast && pos < top_k; ++pos) {
        uint32_t best = 0;
        int bj = 0;
#pragma unroll
        for (int j = 0; j < ITEMS; ++j)
            if (key[j] > best) { // strict: the lowest id of equal keys stays
                best = key[j];
                bj = j;
            }
        const uint32_t top = __reduce_max_sync(0xffffffffu, best);
        float w = 0.0f;
        int id = static_cast<int>(pos); // unfilled slot (qscu.cu:945-949)
        if (top != 0u) {
            const uint32_t cand = best == top ? lane + 32u * static_cast<uint32_t>(bj) : 0xffffffffu;
            const uint32_t win = __reduce_min_sync(0xffffffffu, cand);
            id = static_cast<int>(win);
            const float s = key_score(top);
            w = sigmoid_score ? s : (denom > 0.0f ? expf(s - vmax) / denom : 0.0f);
            if (cand == win) {
#pragma unroll
                for (int j = 0; j < ITEMS; ++j)
                    if (j == bj)
                        key[j] = 0u;
            }
        }
        if (lane == pos) {
            my_weight = w;
            my_id = id;
        }
    }

    float sum = 0.0f;
    for (uint32_t pos = 0; pos < top_k; ++pos)
        sum += __shfl_sync(0xffffffffu, my_weight, pos);
    const float renorm = renormalize ? 1.0f / fmaxf(sum, 1.0e-20f) : 1.0f;
    if (lane < top_k) {
        topk_ids[static_cast<size_t>(token) * top_k + lane] = my_id;
        topk_weights[static_cast<size_t>(token) * top_k + lane] = my_weight * renorm * scaling;
    }
}

// out = bf16(silu(gate) * up); eight elements per thread when aligned.
__global__ void silu_and_mul_kernel(const __nv_bfloat16* __restrict__ gate,
                                    const __nv_bfloat16* __restrict__ up,
                                    __nv_bfloat16* __restrict__ out, uint64_t total, int vec_ok)
{
    const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (vec_ok) {
        const uint64_t i = tid * 8;
        if (i >= total)
            return;
        const uint4 g = *reinterpret_cast<const uint4*>(gate + i);
        const uint4 u = *reinterpret_cast<const uint4*>(up + i);
        const uint32_t gw[4] = { g.x, g.y, g.z, g.w };
        const uint32_t uw[4] = { u.x, u.y, u.z, u.w };
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float g0 = bf16_bits_to_f32(gw[j] & 0xffffu), g1 = bf16_bits_to_f32(gw[j] >> 16);
            const float u0 = bf16_bits_to_f32(uw[j] & 0xffffu), u1 = bf16_bits_to_f32(uw[j] >> 16);
            // upstream qscu.cu:248-251,325: silu(g) = g / (1 + __expf(-g))
            const __nv_bfloat162 r = __floats2bfloat162_rn((g0 / (1.0f + __expf(-g0))) * u0,
                                                           (g1 / (1.0f + __expf(-g1))) * u1);
            ow[j] = *reinterpret_cast<const uint32_t*>(&r);
        }
        *reinterpret_cast<uint4*>(out + i) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    } else {
        if (tid >= total)
            return;
        const float g = __bfloat162float(gate[tid]);
        const float u = __bfloat162float(up[tid]);
        out[tid] = __float2bfloat16((g / (1.0f + __expf(-g))) * u);
    }
}

// out = bf16(f32(out) + sigmoid(gate[t]) * f32(shared)), upstream qscu.cu:338-355.
template <typename GateT>
__global__ void shared_gate_add_kernel(const GateT* __restrict__ gate,
                                       const __nv_bfloat16* __restrict__ shared,
                                       __nv_bfloat16* __restrict__ out, uint32_t hidden,
                                       uint64_t total)
{
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    const uint32_t row = static_cast<uint32_t>(i / hidden);
    float gl;
    if constexpr (sizeof(GateT) == 2)
        gl = __bfloat162float(gate[row]);
    else
        gl = gate[row];
    const float g = sigmoid_fast(gl);
    out[i] = __float2bfloat16(__bfloat162float(out[i]) + g * __bfloat162float(shared[i]));
}

template <typename Tensor> qsfi_status check_tensor(const Tensor& t, qsfi_dtype dtype)
{
    if (t.data == nullptr || t.dtype != dtype)
        return QSFI_STATUS_INVALID_ARGUMENT;
    constexpr uint32_t rank = sizeof(t.shape) / sizeof(t.shape[0]);
    for (uint32_t i = 0; i < rank; ++i)
        if (t.shape[i] <= 0 || t.stride[i] <= 0)
            return QSFI_STATUS_INVALID_ARGUMENT;
    return QSFI_STATUS_OK;
}

template <typename Tensor> qsfi_status check_tensor2(const Tensor& t, qsfi_dtype a, qsfi_dtype b)
{
    if (t.dtype != a && t.dtype != b)
        return QSFI_STATUS_INVALID_ARGUMENT;
    return check_tensor(t, t.dtype);
}

} // namespace

cudaError_t launch_router_topk(const void* logits, int logits_bf16, const float* bias,
                               int32_t* ids, float* weights, uint32_t num_tokens,
                               uint32_t num_experts, uint32_t top_k, int sigmoid_score,
                               int renormalize, float scaling, cudaStream_t stream)
{
    const size_t smem = static_cast<size_t>(kRouterWarps) * num_experts * sizeof(float);
    const uint32_t blocks = (num_tokens + kRouterWarps - 1) / kRouterWarps;
    if (num_experts <= 512) {
        // register-resident variant: ITEMS = experts per lane, rounded up to a power of two
        const uint32_t per_lane = (num_experts + 31) / 32;
#define QS3_ROUTER_REG(T, N)                                                                        \
    router_topk_reg_kernel<T, N><<<blocks, kRouterWarps * 32, 0, stream>>>(                         \
        static_cast<const T*>(logits), bias, ids, weights, num_tokens, num_experts, top_k,          \
        sigmoid_score, renormalize, scaling)
#define QS3_ROUTER_REG_PICK(T)                                                                      \
    do {                                                                                            \
        if (per_lane <= 1)                                                                          \
            QS3_ROUTER_REG(T, 1);                                                                   \
        else if (per_lane <= 2)                                                                     \
            QS3_ROUTER_REG(T, 2);                                                                   \
        else if (per_lane <= 4)                                                                     \
            QS3_ROUTER_REG(T, 4);                                                                   \
        else if (per_lane <= 8)                                                                     \
            QS3_ROUTER_REG(T, 8);                                                                   \
        else                                                                                        \
            QS3_ROUTER_REG(T, 16);                                                                  \
    } while (0)
        if (logits_bf16)
            QS3_ROUTER_REG_PICK(__nv_bfloat16);
        else
            QS3_ROUTER_REG_PICK(float);
#undef QS3_ROUTER_REG_PICK
#undef QS3_ROUTER_REG
        note_launch();
        return cudaGetLastError();
    }
    if (logits_bf16) {
        auto kernel = router_topk_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) {
            cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(smem));
            if (err != cudaSuccess)
                return err;
        }
        kernel<<<blocks, kRouterWarps * 32, smem, stream>>>(
            static_cast<const __nv_bfloat16*>(logits), bias, ids, weights, num_tokens, num_experts,
            top_k, sigmoid_score, renormalize, scaling);
    } else {
        auto kernel = router_topk_kernel<float>;
        if (smem > 48 * 1024) {
            cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(smem));
            if (err != cudaSuccess)
                return err;
        }
        kernel<<<blocks, kRouterWarps * 32, smem, stream>>>(
            static_cast<const float*>(logits), bias, ids, weights, num_tokens, num_experts, top_k,
            sigmoid_score, renormalize, scaling);
    }
    note_launch();
    return cudaGetLastError();
}

// Validation order and status codes of upstream validate_router_desc
// (qscu.cu:1190-1224).
qsfi_status validate_router_desc(const qscu_router_topk_desc* d)
{
    if (d == nullptr || d->num_tokens == 0 || d->num_experts == 0 || d->top_k == 0)
        return QSFI_STATUS_INVALID_ARGUMENT;
    if (d->top_k > kRouterMaxTopK || d->num_experts > kRouterMaxExperts || d->top_k > d->num_experts)
        return QSFI_STATUS_UNSUPPORTED;
    if (d->score != QSCU_ROUTER_SCORE_SOFTMAX && d->score != QSCU_ROUTER_SCORE_SIGMOID)
        return QSFI_STATUS_UNSUPPORTED;
    if (!std::isfinite(d->routed_scaling_factor) || d->routed_scaling_factor <= 0.0f)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qsfi_status s = check_tensor2(d->logits, QSFI_DTYPE_BF16, QSFI_DTYPE_F32);
    if (s != QSFI_STATUS_OK)
        return s;
    s = check_tensor(d->topk_ids, QSFI_DTYPE_I32);
    if (s != QSFI_STATUS_OK)
        return s;
    s = check_tensor(d->topk_weights, QSFI_DTYPE_F32);
    if (s != QSFI_STATUS_OK)
        return s;
    if (!contiguous2(d->logits) || !contiguous2(d->topk_ids) || !contiguous2(d->topk_weights))
        return QSFI_STATUS_INVALID_ARGUMENT;
    if (d->logits.shape[0] != d->num_tokens || d->logits.shape[1] != d->num_experts
        || d->topk_ids.shape[0] != d->num_tokens || d->topk_ids.shape[1] != d->top_k
        || d->topk_weights.shape[0] != d->num_tokens || d->topk_weights.shape[1] != d->top_k)
        return QSFI_STATUS_INVALID_ARGUMENT;
    return QSFI_STATUS_OK;
}

} // namespace qs3

#if QSFI_ENABLE_CHECKED_VALIDATION
namespace qs3 {
namespace {
// upstream validate_finite_tensor2_contents (qscu.cu:158-246): any non-finite logit raises the flag
template <typename T>
__global__ void validate_finite_kernel(const T* v, uint64_t rows, uint64_t cols, int64_t stride0, int64_t stride1,
                                       int* error)
{
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * cols)
        return;
    const int64_t off = static_cast<int64_t>(i / cols) * stride0 + static_cast<int64_t>(i % cols) * stride1;
    if (!isfinite(static_cast<float>(v[off])))
        atomicExch(error, 1);
}
} // namespace
} // namespace qs3
#endif

using namespace qs3;

extern "C" {

qsfi_status qscu_router_topk(const qscu_router_topk_desc* desc, qsfi_cuda_stream stream)
{
    qsfi_status status = validate_router_desc(desc);
    if (status != QSFI_STATUS_OK)
        return status;
#if QSFI_ENABLE_CHECKED_VALIDATION
    {
        // "qscu router logits contain non-finite values" (upstream qscu.cu:1824-1834)
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        cudaError_t verr = cudaSuccess;
        int* flag = checked_flag_reset(st, &verr);
        if (verr != cudaSuccess)
            return status_from_cuda(verr);
        const uint64_t total = static_cast<uint64_t>(desc->num_tokens) * desc->num_experts;
        const uint32_t blocks = static_cast<uint32_t>((total + 255) / 256);
        if (desc->logits.dtype == QSFI_DTYPE_BF16)
            validate_finite_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(desc->logits.data),
                                                          desc->num_tokens, desc->num_experts,
                                                          desc->logits.stride[0], desc->logits.stride[1], flag);
        else
            validate_finite_kernel<<<blocks, 256, 0, st>>>(static_cast<const float*>(desc->logits.data),
                                                          desc->num_tokens, desc->num_experts,
                                                          desc->logits.stride[0], desc->logits.stride[1], flag);
        note_launch();
        verr = cudaGetLastError();
        if (verr != cudaSuccess)
            return status_from_cuda(verr);
        const bool bad = checked_flag_finish(st, &verr);
        if (verr != cudaSuccess)
            return status_from_cuda(verr);
        if (bad)
            return QSFI_STATUS_INVALID_ARGUMENT;
    }
#endif
    cudaError_t err = launch_router_topk(
        desc->logits.data, desc->logits.dtype == QSFI_DTYPE_BF16, nullptr,
        static_cast<int32_t*>(desc->topk_ids.data), static_cast<float*>(desc->topk_weights.data),
        desc->num_tokens, desc->num_experts, desc->top_k,
        desc->score == QSCU_ROUTER_SCORE_SIGMOID, desc->renormalize != 0,
        desc->routed_scaling_factor, static_cast<cudaStream_t>(stream));
    return status_from_cuda(err);
}

// Validation of upstream validate_silu_and_mul_desc (qscu.cu:1226-1253).
qsfi_status qscu_silu_and_mul_bf16(const qscu_silu_and_mul_desc* d, qsfi_cuda_stream stream)
{
    if (d == nullptr || d->num_tokens == 0 || d->intermediate_size == 0)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qsfi_status s = check_tensor(d->gate, QSFI_DTYPE_BF16);
    if (s == QSFI_STATUS_OK)
        s = check_tensor(d->up, QSFI_DTYPE_BF16);
    if (s == QSFI_STATUS_OK)
        s = check_tensor(d->out, QSFI_DTYPE_BF16);
    if (s != QSFI_STATUS_OK)
        return s;
    if (!contiguous2(d->gate) || !contiguous2(d->up) || !contiguous2(d->out))
        return QSFI_STATUS_INVALID_ARGUMENT;
    const int64_t t = d->num_tokens, n = d->intermediate_size;
    if (d->gate.shape[0] != t || d->gate.shape[1] != n || d->up.shape[0] != t
        || d->up.shape[1] != n || d->out.shape[0] != t || d->out.shape[1] != n)
        return QSFI_STATUS_INVALID_ARGUMENT;
    const uint64_t total = static_cast<uint64_t>(t) * static_cast<uint64_t>(n);
    const auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const int vec_ok = total % 8 == 0 && aligned(d->gate.data) && aligned(d->up.data)
        && aligned(d->out.data);
    const uint64_t threads = vec_ok ? total / 8 : total;
    const uint64_t blocks = (threads + 255) / 256;
    if (blocks > 0xffffffffull)
        return QSFI_STATUS_UNSUPPORTED;
    silu_and_mul_kernel<<<static_cast<uint32_t>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(d->gate.data), static_cast<const __nv_bfloat16*>(d->up.data),
        static_cast<__nv_bfloat16*>(d->out.data), total, vec_ok);
    note_launch();
    return status_from_cuda(cudaGetLastError());
}

// Validation of upstream validate_qwen36_shared_expert_gate_add_desc (qscu.cu:1255-1281).
qsfi_status qscu_qwen36_shared_expert_gate_add_bf16(
    const qscu_qwen36_shared_expert_gate_add_desc* d, qsfi_cuda_stream stream)
{
    if (d == nullptr || d->num_tokens == 0 || d->hidden_size == 0)
        return QSFI_STATUS_INVALID_ARGUMENT;
    qsfi_status s = check_tensor2(d->gate_logits, QSFI_DTYPE_BF16, QSFI_DTYPE_F32);
    if (s == QSFI_STATUS_OK)
        s = check_tensor(d->shared, QSFI_DTYPE_BF16);
    if (s == QSFI_STATUS_OK)
        s = check_tensor(d->out, QSFI_DTYPE_BF16);
    if (s != QSFI_STATUS_OK)
        return s;
    if (!contiguous2(d->gate_logits) || !contiguous2(d->shared) || !contiguous2(d->out))
        return QSFI_STATUS_INVALID_ARGUMENT;
    const int64_t t = d->num_tokens, h = d->hidden_size;
    if (d->gate_logits.shape[0] != t || d->gate_logits.shape[1] != 1 || d->shared.shape[0] != t
        || d->shared.shape[1] != h || d->out.shape[0] != t || d->out.shape[1] != h)
        return QSFI_STATUS_INVALID_ARGUMENT;
    const uint64_t total = static_cast<uint64_t>(t) * static_cast<uint64_t>(h);
    const uint64_t blocks = (total + 255) / 256;
    if (blocks > 0xffffffffull)
        return QSFI_STATUS_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d->gate_logits.dtype == QSFI_DTYPE_F32)
        shared_gate_add_kernel<float><<<static_cast<uint32_t>(blocks), 256, 0, st>>>(
            static_cast<const float*>(d->gate_logits.data),
            static_cast<const __nv_bfloat16*>(d->shared.data),
            static_cast<__nv_bfloat16*>(d->out.data), d->hidden_size, total);
    else
        shared_gate_add_kernel<__nv_bfloat16><<<static_cast<uint32_t>(blocks), 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(d->gate_logits.data),
            static_cast<const __nv_bfloat16*>(d->shared.data),
            static_cast<__nv_bfloat16*>(d->out.data), d->hidden_size, total);
    note_launch();
    return status_from_cuda(cudaGetLastError());
}

} // extern "C"
