// Device-side NVFP4 codec: e2m1 codes, one e4m3 scale per 16 elements, one f32
// global scale. The arithmetic (order of operations included) is the same as
// nvfp4_quantize_row in the CPU oracle, so codes can be compared bit for bit:
//   scale = e4m3_rn_sat((amax / 6) / g)
//   code  = e2m1_rn_sat(x * (1 / (f32(scale) * g)))      (0 when scale == 0)
#pragma once

#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace qs3 {

__device__ __forceinline__ uint8_t f32_to_e4m3_sat(float v)
{
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t c)
{
    const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(c), __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&h));
}

// Eight floats -> eight e2m1 codes in one 32-bit word; element i sits in nibble i
// (low nibble = even element). cvt packs its FIRST source into the upper nibble.
__device__ __forceinline__ uint32_t pack_e2m1x8(const float* v)
{
    uint32_t r;
    asm("{\n\t"
        ".reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t"
        "}"
        : "=r"(r)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return r;
}

// Quantise one block of 16 values held by one thread. Returns the scale code and
// writes the 16 codes as two 32-bit words.
__device__ __forceinline__ uint8_t quantize_block16(const float* x, float g, uint32_t* lo, uint32_t* hi)
{
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i)
        amax = fmaxf(amax, fabsf(x[i]));
    // (x / 1 and 1 / s are spelled so that they cost less; both are the same correctly rounded values)
    const float sixth = __fdiv_rn(amax, 6.0f);
    const uint8_t code = f32_to_e4m3_sat(g == 1.0f ? sixth : __fdiv_rn(sixth, g));
    const float s = __fmul_rn(e4m3_to_f32(code), g);
    const float inv = s > 0.0f ? __frcp_rn(s) : 0.0f;
    float q[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
        q[i] = __fmul_rn(x[i], inv);
    *lo = pack_e2m1x8(q);
    *hi = pack_e2m1x8(q + 8);
    return code;
}

// Byte offset of scale (row, kb) in the tiled layout (see include/qs3_moe.h).
__host__ __device__ __forceinline__ uint64_t tiled_scale_offset(uint64_t row, uint64_t kb, uint64_t kgroups)
{
    return ((row >> 7) * kgroups + (kb >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3);
}

// Row of gate_up weight row n in the tiled scale buffer: block j of 128 rows holds
// gate rows [64j, 64j+64) then up rows [inter+64j, inter+64j+64).
__host__ __device__ __forceinline__ uint64_t gated_tiled_row(uint64_t n, uint64_t inter)
{
    const bool up = n >= inter;
    const uint64_t i = up ? n - inter : n;
    return (i >> 6) * 128 + (up ? 64 : 0) + (i & 63);
}

} // namespace qs3
