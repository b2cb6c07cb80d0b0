// qs3_oracle.cpp -- CPU restatement of the qs3 mixture-of-experts path.
//
// TEST INFRASTRUCTURE ONLY. Nothing in the product library links, loads or calls
// this file; it exists so that the CUDA path can be checked against an
// independent host implementation and so that a host-core baseline can be timed.
//
// Each function restates one step of the upstream algorithm and cites the
// upstream file:line it follows. bf16 rounding is applied at every point where
// upstream materialises a bf16 tensor ("strict chain"). The NVFP4 functions
// restate this repository's own quantisation convention (upstream has no NVFP4
// arithmetic: qsfi_moe.cu:807-821 returns UNSUPPORTED), so for those outputs
// parity is unpinned: the oracle and the kernels agree with each other, and no
// upstream value exists to compare against. What IS pinned to a third party is the
// NVFP4 operand format itself: cuBLASLt's block-scaled FP4 GEMM, run on the codes
// and tiled scales the quantisers write, reproduces this file's decode-and-multiply
// (tests/test_gpu_nvfp4_thirdparty.py), and the e4m3 / e2m1 decoders agree with
// torch's dtypes (tests/test_oracle_golden.py).
//
// Parity pins (checked by tests/test_oracle_golden.py): the router known-answer
// cases with ties and non-finite logits (tests_cuda_qscu_gdn_router.inc:966-968,
// :1050; tests_cuda_qscu_utils.inc:733-807), the two hand-computed MoE cases
// (test.cu:1455-1703), the SiLU*mul inputs (tests_cuda_qscu_utils.inc:95-96)
// and the shared-gate inputs (tests_cuda_qscu_utils.inc:144-150).
//
// Build: see oracle/Makefile (g++ -O3 -march=x86-64-v3 -fopenmp -shared).

#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#define QS3O_API extern "C" __attribute__((visibility("default")))

namespace {

// bf16 <- f32, round to nearest even by bit arithmetic, no NaN special case
// (upstream src/model.rs:3000-3004, tests_cuda_qscu_gdn_router.inc:17-24).
inline uint16_t f32_to_bf16(float v)
{
    uint32_t bits;
    std::memcpy(&bits, &v, 4);
    bits += 0x7FFFu + ((bits >> 16) & 1u);
    return static_cast<uint16_t>(bits >> 16);
}

// f32 <- bf16 (upstream test.cu:146-152).
inline float bf16_to_f32(uint16_t b)
{
    uint32_t bits = static_cast<uint32_t>(b) << 16;
    float v;
    std::memcpy(&v, &bits, 4);
    return v;
}

inline float round_bf16(float v)
{
    return bf16_to_f32(f32_to_bf16(v));
}

// upstream qscu.cu:253-256
inline float sigmoidf(float v)
{
    return 1.0f / (1.0f + std::exp(-v));
}

// upstream qscu.cu:248-251
inline float siluf(float v)
{
    return v / (1.0f + std::exp(-v));
}

constexpr float kNegInf = -3.4028234663852886e38f; // upstream qscu.cu:31

// ---- e4m3 / e2m1 codecs (this repository's NVFP4 convention) ----------------

// Unsigned e4m3 decode: 4 exponent bits (bias 7), 3 mantissa bits, max 448.
inline float e4m3_to_f32(uint8_t c)
{
    const int e = (c >> 3) & 0xF;
    const int m = c & 7;
    float v = e == 0 ? std::ldexp(static_cast<float>(m), -9)
                     : std::ldexp(1.0f + static_cast<float>(m) / 8.0f, e - 7);
    return (c & 0x80) ? -v : v;
}

// e4m3 <- f32, round to nearest even, saturate to 448 (no inf/NaN codes are
// produced). Matches cvt.rn.satfinite.e4m3x2.f32 for finite non-negative input.
inline uint8_t f32_to_e4m3(float v)
{
    uint8_t sign = 0;
    if (std::signbit(v)) {
        sign = 0x80;
        v = -v;
    }
    if (!(v == v))
        return static_cast<uint8_t>(sign | 0x7F);
    if (v >= 448.0f)
        return static_cast<uint8_t>(sign | 0x7E);
    if (v < 0.015625f) { // below the smallest normal 2^-6: subnormal step 2^-9
        const float q = std::nearbyint(v * 512.0f); // RNE in default rounding mode
        return static_cast<uint8_t>(sign | static_cast<uint8_t>(q)); // q == 8 -> 0x08 = 2^-6
    }
    int e;
    const float frac = std::frexp(v, &e); // v = frac * 2^e, frac in [0.5, 1)
    // v = (1 + m/8) * 2^(e-1)
    float m = std::nearbyint((frac * 2.0f - 1.0f) * 8.0f);
    int be = e - 1 + 7;
    if (m == 8.0f) {
        m = 0.0f;
        be += 1;
    }
    if (be > 15 || (be == 15 && m > 6.0f))
        return static_cast<uint8_t>(sign | 0x7E);
    return static_cast<uint8_t>(sign | (be << 3) | static_cast<int>(m));
}

const float kE2M1[8] = { 0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f };

// e2m1 <- f32, round to nearest even (ties go to the code with even mantissa
// bit), saturate to 6. Matches cvt.rn.satfinite.e2m1x2.f32 for finite input.
inline uint8_t f32_to_e2m1(float v)
{
    uint8_t sign = 0;
    if (std::signbit(v)) {
        sign = 8;
        v = -v;
    }
    uint8_t c;
    if (!(v == v))
        c = 7;
    else if (v <= 0.25f)
        c = 0;
    else if (v < 0.75f)
        c = 1;
    else if (v <= 1.25f)
        c = 2;
    else if (v < 1.75f)
        c = 3;
    else if (v <= 2.5f)
        c = 4;
    else if (v < 3.5f)
        c = 5;
    else if (v <= 5.0f)
        c = 6;
    else
        c = 7;
    return static_cast<uint8_t>(sign | c);
}

inline float e2m1_to_f32(uint8_t c)
{
    const float v = kE2M1[c & 7];
    return (c & 8) ? -v : v;
}

// Quantise one row of k floats: per 16-element block, scale = e4m3(amax / 6 / g),
// code = e2m1(x * (1 / (f32(scale) * g))). packed: low nibble = even k.
void nvfp4_quantize_row(const float* x, int64_t k, float g, uint8_t* packed, uint8_t* scales)
{
    for (int64_t b = 0; b < k / 16; ++b) {
        float amax = 0.0f;
        for (int i = 0; i < 16; ++i)
            amax = std::fmax(amax, std::fabs(x[b * 16 + i]));
        const uint8_t sc = f32_to_e4m3((amax / 6.0f) / g);
        scales[b] = sc;
        const float s = e4m3_to_f32(sc) * g;
        const float inv = s > 0.0f ? 1.0f / s : 0.0f;
        for (int i = 0; i < 16; i += 2) {
            const uint8_t lo = f32_to_e2m1(x[b * 16 + i] * inv);
            const uint8_t hi = f32_to_e2m1(x[b * 16 + i + 1] * inv);
            packed[b * 8 + i / 2] = static_cast<uint8_t>(lo | (hi << 4));
        }
    }
}

// Dequantise one row to floats WITHOUT the global scale (code * block scale).
void nvfp4_dequantize_row(const uint8_t* packed, const uint8_t* scales, int64_t k, float* out)
{
    for (int64_t b = 0; b < k / 16; ++b) {
        const float s = e4m3_to_f32(scales[b]);
        for (int i = 0; i < 8; ++i) {
            const uint8_t byte = packed[b * 8 + i];
            out[b * 16 + 2 * i] = e2m1_to_f32(byte & 0xF) * s;
            out[b * 16 + 2 * i + 1] = e2m1_to_f32(byte >> 4) * s;
        }
    }
}

inline float dotf(const float* a, const float* b, int64_t n)
{
    float acc = 0.0f;
#pragma omp simd reduction(+ : acc)
    for (int64_t i = 0; i < n; ++i)
        acc += a[i] * b[i];
    return acc;
}

// Offset of scale (row, kblock) in the tiled layout described in include/qs3_moe.h.
inline int64_t tiled_scale_offset(int64_t row, int64_t kb, int64_t k)
{
    const int64_t kgroups = k / 64;
    return ((row / 128) * kgroups + kb / 4) * 512 + (row % 32) * 16 + ((row / 32) % 4) * 4 + kb % 4;
}

// Row order of the gate_up tiled-scale buffer: 128-row block j holds gate rows
// [64j, 64j+64) followed by up rows [inter+64j, inter+64j+64).
inline int64_t gated_tiled_row(int64_t n, int64_t inter)
{
    const bool up = n >= inter;
    const int64_t i = up ? n - inter : n;
    return (i / 64) * 128 + (up ? 64 : 0) + i % 64;
}

} // namespace

// ------------------------------------------------------------------ codecs ---

QS3O_API uint16_t qs3o_f32_to_bf16(float v) { return f32_to_bf16(v); }
QS3O_API float qs3o_bf16_to_f32(uint16_t b) { return bf16_to_f32(b); }
QS3O_API uint8_t qs3o_f32_to_e4m3(float v) { return f32_to_e4m3(v); }
QS3O_API float qs3o_e4m3_to_f32(uint8_t c) { return e4m3_to_f32(c); }
QS3O_API uint8_t qs3o_f32_to_e2m1(float v) { return f32_to_e2m1(v); }
QS3O_API float qs3o_e2m1_to_f32(uint8_t c) { return e2m1_to_f32(c); }
QS3O_API int qs3o_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Number of OpenMP threads later calls use (launchers such as torch.distributed.run export
// OMP_NUM_THREADS=1, which would otherwise time this code on one core).
QS3O_API void qs3o_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// ------------------------------------------------------------------ router ---

// Router top-k for one block of tokens. Follows the upstream CPU checker
// (tests_cuda_qscu_gdn_router.inc:223-292) and, where the two differ, the device
// kernel (qscu.cu:894-971): unfilled slots (possible only with NaN / -inf
// logits) become id = slot index with weight 0 (qscu.cu:945-949), and a softmax
// denominator that is not > 0 gives weight 0 (qscu.cu:953).
// `bias` (optional, f32[num_experts]) is added to the f32 logits first; it is
// this repository's additive router_bias input and NULL reproduces upstream.
QS3O_API void qs3o_router_topk(
    const float* logits, int64_t num_tokens, int64_t num_experts, int64_t top_k, int score,
    int renormalize, float scaling, const float* bias, int32_t* ids, float* weights
)
{
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < num_tokens; ++t) {
        std::vector<float> row(num_experts);
        for (int64_t e = 0; e < num_experts; ++e)
            row[e] = logits[t * num_experts + e] + (bias ? bias[e] : 0.0f);

        float max_logit = kNegInf;
        float denom = 0.0f;
        if (score == 0) {
            for (int64_t e = 0; e < num_experts; ++e)
                if (row[e] > max_logit)
                    max_logit = row[e];
            for (int64_t e = 0; e < num_experts; ++e)
                denom += std::exp(row[e] - max_logit);
        }

        float best[16];
        int32_t best_id[16];
        for (int p = 0; p < 16; ++p) {
            best[p] = kNegInf;
            best_id[p] = INT_MAX;
        }
        for (int64_t e = 0; e < num_experts; ++e) {
            const float s = score == 0 ? row[e] : sigmoidf(row[e]);
            for (int64_t p = 0; p < top_k; ++p) {
                const bool better = s > best[p] || (s == best[p] && e < best_id[p]);
                if (!better)
                    continue;
                for (int64_t m = top_k - 1; m > p; --m) {
                    best[m] = best[m - 1];
                    best_id[m] = best_id[m - 1];
                }
                best[p] = s;
                best_id[p] = static_cast<int32_t>(e);
                break;
            }
        }

        float sum = 0.0f;
        float w[16];
        for (int64_t p = 0; p < top_k; ++p) {
            if (best_id[p] == INT_MAX) {
                best_id[p] = static_cast<int32_t>(p);
                w[p] = 0.0f;
                continue;
            }
            const float l = row[best_id[p]];
            w[p] = score == 0 ? (denom > 0.0f ? std::exp(l - max_logit) / denom : 0.0f)
                              : sigmoidf(l);
            sum += w[p];
        }
        const float renorm = renormalize ? 1.0f / std::fmax(sum, 1.0e-20f) : 1.0f;
        for (int64_t p = 0; p < top_k; ++p) {
            ids[t * top_k + p] = best_id[p];
            weights[t * top_k + p] = w[p] * renorm * scaling;
        }
    }
}

// --------------------------------------------------------- route permutation ---

// Histogram, exclusive scan and route -> row placement (upstream
// qsfi_moe.cu:327-386). Upstream places rows inside an expert segment in
// atomics order; the canonical order used here and by the CUDA path is stable
// in route index (route = token * top_k + k). Non-local routes get row -1.
QS3O_API void qs3o_route_sort(
    const int32_t* ids, const float* weights, int64_t num_tokens, int64_t top_k,
    int64_t local_offset, int64_t local_experts, int32_t* counts, int32_t* indptr,
    int32_t* route_rows, int32_t* row_tokens, float* row_scales
)
{
    const int64_t routes = num_tokens * top_k;
    std::fill(counts, counts + local_experts, 0);
    for (int64_t r = 0; r < routes; ++r) {
        const int64_t local = static_cast<int64_t>(ids[r]) - local_offset;
        if (local >= 0 && local < local_experts)
            counts[local] += 1;
    }
    indptr[0] = 0;
    for (int64_t e = 0; e < local_experts; ++e)
        indptr[e + 1] = indptr[e] + counts[e];
    std::vector<int32_t> cursor(indptr, indptr + local_experts);
    for (int64_t r = 0; r < routes; ++r) {
        const int64_t local = static_cast<int64_t>(ids[r]) - local_offset;
        if (local < 0 || local >= local_experts) {
            route_rows[r] = -1;
            continue;
        }
        const int32_t row = cursor[local]++;
        route_rows[r] = row;
        row_tokens[row] = static_cast<int32_t>(r / top_k);
        row_scales[row] = weights[r];
    }
}

// ------------------------------------------------------------- element-wise ---

// upstream qscu.cu:306-327: out = bf16(silu(gate) * up)
QS3O_API void
qs3o_silu_and_mul_bf16(const uint16_t* gate, const uint16_t* up, int64_t n, uint16_t* out)
{
    for (int64_t i = 0; i < n; ++i)
        out[i] = f32_to_bf16(siluf(bf16_to_f32(gate[i])) * bf16_to_f32(up[i]));
}

// upstream qscu.cu:338-355: out = bf16(f32(out) + sigmoid(gate[t]) * f32(shared))
QS3O_API void qs3o_shared_gate_add_bf16(
    const float* gate_logits, const uint16_t* shared, int64_t num_tokens, int64_t hidden,
    uint16_t* out
)
{
    for (int64_t t = 0; t < num_tokens; ++t) {
        const float g = sigmoidf(gate_logits[t]);
        for (int64_t h = 0; h < hidden; ++h) {
            const int64_t i = t * hidden + h;
            out[i] = f32_to_bf16(bf16_to_f32(out[i]) + g * bf16_to_f32(shared[i]));
        }
    }
}

// Dense GEMM semantics of upstream qscb.h:14-25 (CPU dot in
// tests_cuda_qscb_gemm.inc:43-61): out[r, o] = alpha * sum_i x[r, i] * w[o, i]
// + beta * out[r, o], f32 accumulation; out is f32 (out_f32 != NULL) or bf16.
QS3O_API void qs3o_gemm_bf16(
    const uint16_t* x, const uint16_t* w, int64_t rows, int64_t in_features, int64_t out_features,
    float alpha, float beta, float* out_f32, uint16_t* out_bf16
)
{
    std::vector<float> xf(rows * in_features);
    for (int64_t i = 0; i < rows * in_features; ++i)
        xf[i] = bf16_to_f32(x[i]);
#pragma omp parallel
    {
        std::vector<float> wf(in_features);
#pragma omp for schedule(static)
        for (int64_t o = 0; o < out_features; ++o) {
            for (int64_t i = 0; i < in_features; ++i)
                wf[i] = bf16_to_f32(w[o * in_features + i]);
            for (int64_t r = 0; r < rows; ++r) {
                float acc = alpha * dotf(&xf[r * in_features], wf.data(), in_features);
                const int64_t idx = r * out_features + o;
                if (out_f32) {
                    if (beta != 0.0f)
                        acc += beta * out_f32[idx];
                    out_f32[idx] = acc;
                } else {
                    if (beta != 0.0f)
                        acc += beta * bf16_to_f32(out_bf16[idx]);
                    out_bf16[idx] = f32_to_bf16(acc);
                }
            }
        }
    }
}

// ---------------------------------------------------------------- bf16 MoE ---

// Routed experts in bf16, strict chain (upstream qsfi_moe.cu:539-724):
//   Y1 = bf16(X * Wgu^T)            grouped GEMM, f32 accumulate, bf16 store
//   act = bf16(g * sigmoid(g) * u)  qsfi_moe.cu:459-462, g/u read back from bf16 Y1
//   Y2 = bf16(act * Wd^T)
//   out[t] = bf16(sum_k w[t,k] * f32(Y2[row(t,k)]))   k ascending, qsfi_moe.cu:481-491
// Tokens are independent, so the computation is organised per token; `token_list`
// (optional, n_list entries) restricts the work to those tokens and `out` then has
// n_list rows. Non-local routes are skipped (qsfi_moe.cu:484).
QS3O_API void qs3o_moe_bf16(
    const uint16_t* hidden, const int32_t* ids, const float* weights, const uint16_t* gate_up,
    const uint16_t* down, int64_t num_tokens, int64_t hidden_size, int64_t inter, int64_t top_k,
    int64_t local_offset, int64_t local_experts, const int32_t* token_list, int64_t n_list,
    uint16_t* out
)
{
    const int64_t n = token_list ? n_list : num_tokens;
#pragma omp parallel
    {
        std::vector<float> x(hidden_size), y1(2 * inter), act(inter), wrow(std::max(hidden_size, inter)),
            acc(hidden_size);
#pragma omp for schedule(dynamic, 1)
        for (int64_t li = 0; li < n; ++li) {
            const int64_t t = token_list ? token_list[li] : li;
            for (int64_t h = 0; h < hidden_size; ++h)
                x[h] = bf16_to_f32(hidden[t * hidden_size + h]);
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (int64_t k = 0; k < top_k; ++k) {
                const int64_t local = static_cast<int64_t>(ids[t * top_k + k]) - local_offset;
                if (local < 0 || local >= local_experts)
                    continue;
                const float wgt = weights[t * top_k + k];
                const uint16_t* wgu = gate_up + local * 2 * inter * hidden_size;
                for (int64_t j = 0; j < 2 * inter; ++j) {
                    for (int64_t h = 0; h < hidden_size; ++h)
                        wrow[h] = bf16_to_f32(wgu[j * hidden_size + h]);
                    y1[j] = round_bf16(dotf(x.data(), wrow.data(), hidden_size));
                }
                for (int64_t i = 0; i < inter; ++i) {
                    const float g = y1[i];
                    const float u = y1[inter + i];
                    act[i] = round_bf16(g * (1.0f / (1.0f + std::exp(-g))) * u);
                }
                const uint16_t* wd = down + local * hidden_size * inter;
                for (int64_t h = 0; h < hidden_size; ++h) {
                    for (int64_t i = 0; i < inter; ++i)
                        wrow[i] = bf16_to_f32(wd[h * inter + i]);
                    const float y2 = round_bf16(dotf(act.data(), wrow.data(), inter));
                    acc[h] += wgt * y2;
                }
            }
            for (int64_t h = 0; h < hidden_size; ++h)
                out[li * hidden_size + h] = f32_to_bf16(acc[h]);
        }
    }
}

// Shared expert in bf16, strict chain (upstream src/model.rs:2174-2228):
//   g = bf16(x Wg^T), u = bf16(x Wu^T), mlp = bf16(silu(g) * u), s = bf16(mlp Wd^T),
//   gamma = f32(x wgate^T), out = bf16(f32(out) + sigmoid(gamma) * f32(s)).
// `gate_up` is [2*Is, H] with gate rows first. `out` is updated in place and has
// one row per listed token.
QS3O_API void qs3o_shared_expert_bf16(
    const uint16_t* hidden, const uint16_t* gate_up, const uint16_t* down, const uint16_t* gate_w,
    int64_t num_tokens, int64_t hidden_size, int64_t inter, const int32_t* token_list,
    int64_t n_list, uint16_t* out
)
{
    const int64_t n = token_list ? n_list : num_tokens;
#pragma omp parallel
    {
        std::vector<float> x(hidden_size), y1(2 * inter), mlp(inter), wrow(std::max(hidden_size, inter));
#pragma omp for schedule(dynamic, 1)
        for (int64_t li = 0; li < n; ++li) {
            const int64_t t = token_list ? token_list[li] : li;
            for (int64_t h = 0; h < hidden_size; ++h)
                x[h] = bf16_to_f32(hidden[t * hidden_size + h]);
            for (int64_t j = 0; j < 2 * inter; ++j) {
                for (int64_t h = 0; h < hidden_size; ++h)
                    wrow[h] = bf16_to_f32(gate_up[j * hidden_size + h]);
                y1[j] = round_bf16(dotf(x.data(), wrow.data(), hidden_size));
            }
            for (int64_t i = 0; i < inter; ++i)
                mlp[i] = round_bf16(siluf(y1[i]) * y1[inter + i]);
            for (int64_t h = 0; h < hidden_size; ++h)
                wrow[h] = bf16_to_f32(gate_w[h]);
            const float gamma = sigmoidf(dotf(x.data(), wrow.data(), hidden_size));
            for (int64_t h = 0; h < hidden_size; ++h) {
                for (int64_t i = 0; i < inter; ++i)
                    wrow[i] = bf16_to_f32(down[h * inter + i]);
                const float s = round_bf16(dotf(mlp.data(), wrow.data(), inter));
                const int64_t idx = li * hidden_size + h;
                out[idx] = f32_to_bf16(bf16_to_f32(out[idx]) + gamma * s);
            }
        }
    }
}

// ------------------------------------------------------------------- NVFP4 ---

QS3O_API int64_t qs3o_tiled_scale_bytes(int64_t rows, int64_t k)
{
    return ((rows + 127) / 128) * (k / 64) * 512;
}

QS3O_API int64_t qs3o_tiled_scale_offset(int64_t row, int64_t kb, int64_t k)
{
    return tiled_scale_offset(row, kb, k);
}

QS3O_API int64_t qs3o_gated_tiled_row(int64_t n, int64_t inter)
{
    return gated_tiled_row(n, inter);
}

// Quantise activations (bf16 rows) with a given global scale; linear scale layout.
QS3O_API void qs3o_nvfp4_quantize_act(
    const uint16_t* x, int64_t rows, int64_t k, float global_scale, uint8_t* packed,
    uint8_t* scale_linear
)
{
    const float g = global_scale == 0.0f ? 1.0f : global_scale;
#pragma omp parallel
    {
        std::vector<float> xf(k);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            for (int64_t i = 0; i < k; ++i)
                xf[i] = bf16_to_f32(x[r * k + i]);
            nvfp4_quantize_row(xf.data(), k, g, packed + r * (k / 2), scale_linear + r * (k / 16));
        }
    }
}

// Quantise expert weights bf16 [experts, rows, k]: global[e] = amax_e / (6 * 448)
// (1 when the expert is all zero); block scales in the linear layout and, when
// scale_tiled != NULL, also in the tiled layout (gated != 0: gate_up row order).
QS3O_API void qs3o_nvfp4_quantize_weight(
    const uint16_t* w, int64_t experts, int64_t rows, int64_t k, int gated, uint8_t* packed,
    uint8_t* scale_linear, uint8_t* scale_tiled, float* global_scale
)
{
    const int64_t tiled_bytes = qs3o_tiled_scale_bytes(rows, k);
    for (int64_t e = 0; e < experts; ++e) {
        const uint16_t* we = w + e * rows * k;
        float amax = 0.0f;
#pragma omp parallel for reduction(max : amax) schedule(static)
        for (int64_t i = 0; i < rows * k; ++i)
            amax = std::fmax(amax, std::fabs(bf16_to_f32(we[i])));
        const float g = amax > 0.0f ? amax / (6.0f * 448.0f) : 1.0f;
        global_scale[e] = g;
#pragma omp parallel
        {
            std::vector<float> xf(k);
            std::vector<uint8_t> sc(k / 16);
#pragma omp for schedule(static)
            for (int64_t r = 0; r < rows; ++r) {
                for (int64_t i = 0; i < k; ++i)
                    xf[i] = bf16_to_f32(we[r * k + i]);
                nvfp4_quantize_row(xf.data(), k, g, packed + (e * rows + r) * (k / 2), sc.data());
                if (scale_linear)
                    std::memcpy(scale_linear + (e * rows + r) * (k / 16), sc.data(), k / 16);
                if (scale_tiled) {
                    const int64_t tr = gated ? gated_tiled_row(r, rows / 2) : r;
                    for (int64_t b = 0; b < k / 16; ++b)
                        scale_tiled[e * tiled_bytes + tiled_scale_offset(tr, b, k)] = sc[b];
                }
            }
        }
    }
}

// Routed + optional shared experts on NVFP4 operands, this repository's chain:
//   xq = quantise(x, act_global)                       (or given pre-quantised)
//   Y1 = (xq . Wgu_q) * act_global * gu_global[e]      f32, no bf16 rounding; with bit 0 of gu_split
//        set gu_global holds [2, experts]: row 0 scales the gate rows, row 1 the up rows
//        (bit 1: the same for the shared expert, sh_gu_global = [gate, up])
//   act = g * sigmoid(g) * u                           f32
//   aq = quantise(act, act2_global)
//   Y2 = bf16((aq . Wd_q) * act2_global * d_global[e])
//   out[t] = bf16(sum_k w[t,k] * f32(Y2) [+ sigmoid(x . wgate) * f32(Y2_shared)])
// Weight scales are read from the LINEAR layout. hidden_packed/hidden_scale are
// the already-quantised activations [T, H/2] / [T, H/16]. For the shared expert
// pass shared_* (experts = 1) and gate_w bf16[H] with hidden_bf16 (needed for the
// gate logit); otherwise NULL.
QS3O_API void qs3o_moe_nvfp4(
    const uint8_t* hidden_packed, const uint8_t* hidden_scale, float act_global, float act2_global,
    const int32_t* ids, const float* weights, const uint8_t* gu_packed, const uint8_t* gu_scale,
    const float* gu_global, const uint8_t* d_packed, const uint8_t* d_scale, const float* d_global,
    int64_t num_tokens, int64_t hidden_size, int64_t inter, int64_t top_k, int64_t local_offset,
    int64_t local_experts, const uint8_t* sh_gu_packed, const uint8_t* sh_gu_scale,
    const float* sh_gu_global, const uint8_t* sh_d_packed, const uint8_t* sh_d_scale,
    const float* sh_d_global, int64_t shared_inter, const uint16_t* hidden_bf16,
    const uint16_t* gate_w, const int32_t* token_list, int64_t n_list, int32_t gu_split, uint16_t* out
)
{
    const float ga = act_global == 0.0f ? 1.0f : act_global;
    const float ga2 = act2_global == 0.0f ? 1.0f : act2_global;
    const int64_t n = token_list ? n_list : num_tokens;
    const int64_t max_inter = std::max(inter, shared_inter);
#pragma omp parallel
    {
        std::vector<float> x(hidden_size), y1(2 * max_inter), act(max_inter), aq(max_inter),
            wrow(std::max(hidden_size, max_inter)), acc(hidden_size), xb(hidden_size);
        std::vector<uint8_t> ap(max_inter / 2), as(max_inter / 16);

        auto run_expert = [&](const uint8_t* gup, const uint8_t* gus, float gug, float gug_up,
                              const uint8_t* dp, const uint8_t* ds, float dg, int64_t I, float wgt) {
            for (int64_t j = 0; j < 2 * I; ++j) {
                nvfp4_dequantize_row(gup + j * (hidden_size / 2), gus + j * (hidden_size / 16),
                                     hidden_size, wrow.data());
                y1[j] = dotf(x.data(), wrow.data(), hidden_size) * (ga * (j < I ? gug : gug_up));
            }
            for (int64_t i = 0; i < I; ++i) {
                const float g = y1[i];
                act[i] = g * (1.0f / (1.0f + std::exp(-g))) * y1[I + i];
            }
            nvfp4_quantize_row(act.data(), I, ga2, ap.data(), as.data());
            nvfp4_dequantize_row(ap.data(), as.data(), I, aq.data());
            for (int64_t h = 0; h < hidden_size; ++h) {
                nvfp4_dequantize_row(dp + h * (I / 2), ds + h * (I / 16), I, wrow.data());
                const float y2 = round_bf16(dotf(aq.data(), wrow.data(), I) * (ga2 * dg));
                acc[h] += wgt * y2;
            }
        };

#pragma omp for schedule(dynamic, 1)
        for (int64_t li = 0; li < n; ++li) {
            const int64_t t = token_list ? token_list[li] : li;
            nvfp4_dequantize_row(hidden_packed + t * (hidden_size / 2),
                                 hidden_scale + t * (hidden_size / 16), hidden_size, x.data());
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (int64_t k = 0; k < top_k; ++k) {
                const int64_t local = static_cast<int64_t>(ids[t * top_k + k]) - local_offset;
                if (local < 0 || local >= local_experts)
                    continue;
                run_expert(gu_packed + local * 2 * inter * (hidden_size / 2),
                           gu_scale + local * 2 * inter * (hidden_size / 16), gu_global[local],
                           gu_global[(gu_split & 1) ? local_experts + local : local],
                           d_packed + local * hidden_size * (inter / 2),
                           d_scale + local * hidden_size * (inter / 16), d_global[local], inter,
                           weights[t * top_k + k]);
            }
            if (sh_gu_packed) {
                for (int64_t h = 0; h < hidden_size; ++h) {
                    xb[h] = bf16_to_f32(hidden_bf16[t * hidden_size + h]);
                    wrow[h] = bf16_to_f32(gate_w[h]);
                }
                const float gamma = sigmoidf(dotf(xb.data(), wrow.data(), hidden_size));
                run_expert(sh_gu_packed, sh_gu_scale, sh_gu_global[0], sh_gu_global[(gu_split & 2) ? 1 : 0],
                           sh_d_packed, sh_d_scale,
                           sh_d_global[0], shared_inter, gamma);
            }
            for (int64_t h = 0; h < hidden_size; ++h)
                out[li * hidden_size + h] = f32_to_bf16(acc[h]);
        }
    }
}

// ---- FP8 block-scaled path (this repository's convention; upstream has no FP8 MoE
// surface at all, only the dtype enum values in qs_tensor.h:20-24, so parity is
// unpinned here as well) --------------------------------------------------------------
//   activations: e4m3 codes, one f32 scale per token per 128 consecutive elements
//   weights:     e4m3 codes, one f32 scale per 128 x 128 block (rows x k)
//   scale = max(amax / 448, 1e-30);  code = e4m3_rn_sat(x * (1 / scale))

namespace {

inline float fp8_scale(float amax)
{
    return std::max(amax / 448.0f, 1.0e-30f);
}

void fp8_quantize_group(const float* x, int64_t n, uint8_t* codes, float* scale)
{
    float amax = 0.0f;
    for (int64_t i = 0; i < n; ++i)
        amax = std::max(amax, std::fabs(x[i]));
    const float s = fp8_scale(amax);
    const float inv = 1.0f / s;
    for (int64_t i = 0; i < n; ++i)
        codes[i] = f32_to_e4m3(x[i] * inv);
    *scale = s;
}

// y[j] = sum_kb (a_scale[kb] * w_scale[j / 128][kb]) * sum_{k in kb} a[k] * w[j][k]
// for rows j of one expert matrix [rows, k]; the inner sums are exact (double).
void fp8_matvec(const uint8_t* a, const float* a_scale, const uint8_t* w, const float* w_scale,
                int64_t rows, int64_t k, const float* lut, float* y)
{
    const int64_t kb_n = k / 128;
    for (int64_t j = 0; j < rows; ++j) {
        const uint8_t* wr = w + j * k;
        const float* ws = w_scale + (j / 128) * kb_n;
        float acc = 0.0f;
        for (int64_t kb = 0; kb < kb_n; ++kb) {
            double part = 0.0;
            for (int64_t i = kb * 128; i < (kb + 1) * 128; ++i)
                part += static_cast<double>(lut[a[i]]) * static_cast<double>(lut[wr[i]]);
            acc += static_cast<float>(part) * (ws[kb] * a_scale[kb]);
        }
        y[j] = acc;
    }
}

} // namespace

// codes u8 [rows, k], scales f32 [rows, k / 128]; k % 128 == 0.
QS3O_API void
qs3o_fp8_quantize_act(const uint16_t* x, int64_t rows, int64_t k, uint8_t* codes, float* scales)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float v[128];
        for (int64_t g = 0; g < k / 128; ++g) {
            for (int64_t i = 0; i < 128; ++i)
                v[i] = bf16_to_f32(x[r * k + g * 128 + i]);
            fp8_quantize_group(v, 128, codes + r * k + g * 128, scales + r * (k / 128) + g);
        }
    }
}

// codes u8 [experts, rows, k], scales f32 [experts, ceil(rows / 128), k / 128].
QS3O_API void qs3o_fp8_quantize_weight(
    const uint16_t* w, int64_t experts, int64_t rows, int64_t k, uint8_t* codes, float* scales
)
{
    const int64_t rb_n = (rows + 127) / 128, kb_n = k / 128;
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t e = 0; e < experts; ++e) {
        for (int64_t rb = 0; rb < rb_n; ++rb) {
            const int64_t r1 = std::min(rows, (rb + 1) * 128);
            for (int64_t kb = 0; kb < kb_n; ++kb) {
                float amax = 0.0f;
                for (int64_t r = rb * 128; r < r1; ++r)
                    for (int64_t i = kb * 128; i < (kb + 1) * 128; ++i)
                        amax = std::max(amax, std::fabs(bf16_to_f32(w[(e * rows + r) * k + i])));
                const float s = fp8_scale(amax);
                const float inv = 1.0f / s;
                for (int64_t r = rb * 128; r < r1; ++r)
                    for (int64_t i = kb * 128; i < (kb + 1) * 128; ++i)
                        codes[(e * rows + r) * k + i]
                            = f32_to_e4m3(bf16_to_f32(w[(e * rows + r) * k + i]) * inv);
                scales[(e * rb_n + rb) * kb_n + kb] = s;
            }
        }
    }
}

// Routed experts on FP8 operands, this repository's chain:
//   Y1 = blockscaled(xq . Wgu_q)            f32, no bf16 rounding
//   act = g * sigmoid(g) * u                f32
//   aq = quantise(act) per token per 128 features
//   Y2 = bf16(blockscaled(aq . Wd_q))
//   out[t] = bf16(sum_k w[t,k] * f32(Y2))
QS3O_API void qs3o_moe_fp8(
    const uint8_t* hidden_codes, const float* hidden_scale, const int32_t* ids, const float* weights,
    const uint8_t* gu_codes, const float* gu_scale, const uint8_t* d_codes, const float* d_scale,
    int64_t num_tokens, int64_t hidden_size, int64_t inter, int64_t top_k, int64_t local_offset,
    int64_t local_experts, const int32_t* token_list, int64_t n_list, uint16_t* out
)
{
    float lut[256];
    for (int c = 0; c < 256; ++c)
        lut[c] = e4m3_to_f32(static_cast<uint8_t>(c));
    const int64_t n = token_list ? n_list : num_tokens;
    const int64_t hb = hidden_size / 128, ib = inter / 128, gub = (2 * inter + 127) / 128;
#pragma omp parallel
    {
        std::vector<float> y1(2 * inter), act(inter), as(ib), y2(hidden_size), acc(hidden_size);
        std::vector<uint8_t> aq(inter);
#pragma omp for schedule(dynamic, 1)
        for (int64_t li = 0; li < n; ++li) {
            const int64_t t = token_list ? token_list[li] : li;
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (int64_t k = 0; k < top_k; ++k) {
                const int64_t local = static_cast<int64_t>(ids[t * top_k + k]) - local_offset;
                if (local < 0 || local >= local_experts)
                    continue;
                fp8_matvec(hidden_codes + t * hidden_size, hidden_scale + t * hb,
                           gu_codes + local * 2 * inter * hidden_size, gu_scale + local * gub * hb,
                           2 * inter, hidden_size, lut, y1.data());
                for (int64_t i = 0; i < inter; ++i) {
                    const float g = y1[i];
                    act[i] = g * (1.0f / (1.0f + std::exp(-g))) * y1[inter + i];
                }
                for (int64_t g = 0; g < ib; ++g)
                    fp8_quantize_group(act.data() + g * 128, 128, aq.data() + g * 128, as.data() + g);
                fp8_matvec(aq.data(), as.data(), d_codes + local * hidden_size * inter,
                           d_scale + local * hb * ib, hidden_size, inter, lut, y2.data());
                const float wgt = weights[t * top_k + k];
                for (int64_t h = 0; h < hidden_size; ++h)
                    acc[h] += wgt * round_bf16(y2[h]);
            }
            for (int64_t h = 0; h < hidden_size; ++h)
                out[li * hidden_size + h] = f32_to_bf16(acc[h]);
        }
    }
}

// ---- RMSNorm neighbours of the MoE block ---------------------------------------------------
// Restates the upstream CPU checkers of the FlashInfer-backed norms
// (tests_cuda_flashinfer_norm_rope.inc:139-188 and :190-246): everything in f32, the sum of
// squares in column order, inv_rms = 1 / sqrt(sum / hidden + eps), plain weight (+ bias).
// Inputs are bf16 bit patterns (is_bf16 != 0) or f32; outputs are f32 (the device result is
// compared within the tolerances of the upstream tests: f32 2e-5 / 1e-5, bf16 0.018 / 0.012).

namespace {
inline float load_elem(const void* p, int is_bf16, int64_t i)
{
    return is_bf16 ? bf16_to_f32(static_cast<const uint16_t*>(p)[i]) : static_cast<const float*>(p)[i];
}
} // namespace

QS3O_API void qs3o_rmsnorm(
    const void* x, const void* weight, int is_bf16, int64_t rows, int64_t hidden, float eps,
    float weight_bias, float* out
)
{
    for (int64_t r = 0; r < rows; ++r) {
        float sum_sq = 0.0f;
        for (int64_t c = 0; c < hidden; ++c) {
            const float v = load_elem(x, is_bf16, r * hidden + c);
            sum_sq += v * v;
        }
        const float inv_rms = 1.0f / std::sqrt(sum_sq / static_cast<float>(hidden) + eps);
        for (int64_t c = 0; c < hidden; ++c)
            out[r * hidden + c]
                = load_elem(x, is_bf16, r * hidden + c) * inv_rms * (weight_bias + load_elem(weight, is_bf16, c));
    }
}

QS3O_API void qs3o_fused_add_rmsnorm(
    const void* x, const void* residual, const void* weight, int is_bf16, int64_t rows,
    int64_t hidden, float eps, float* norm_out, float* residual_out
)
{
    for (int64_t r = 0; r < rows; ++r) {
        float sum_sq = 0.0f;
        for (int64_t c = 0; c < hidden; ++c) {
            const float v = load_elem(x, is_bf16, r * hidden + c) + load_elem(residual, is_bf16, r * hidden + c);
            residual_out[r * hidden + c] = v;
            sum_sq += v * v;
        }
        const float inv_rms = 1.0f / std::sqrt(sum_sq / static_cast<float>(hidden) + eps);
        for (int64_t c = 0; c < hidden; ++c)
            norm_out[r * hidden + c] = residual_out[r * hidden + c] * inv_rms * load_elem(weight, is_bf16, c);
    }
}
