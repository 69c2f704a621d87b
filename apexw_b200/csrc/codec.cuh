// Device-side storage codecs: bf16 stochastic rounding, NF4, log-uint8.
// Formats are defined in apexw_b200/ops/formats.py; the arithmetic here follows
// that file operation by operation (this translation unit is compiled with
// -fmad=false so that products and sums round separately, as torch does).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include "plan_types.h"

namespace apexb {


__device__ __forceinline__ float bf16_bits_to_float(uint32_t hi16) { return __uint_as_float(hi16 << 16); }

// NaN -> 0, +-Inf -> +-65504 (what torch.nan_to_num(g, 0, 65504, -65504) does)
__device__ __forceinline__ float sanitize_grad(float g) {
    const uint32_t u = __float_as_uint(g);
    if ((u & 0x7F800000u) == 0x7F800000u) {
        if (u & 0x007FFFFFu) return 0.0f;
        return (u >> 31) ? -65504.0f : 65504.0f;
    }
    return g;
}

// NF4 codes of two values x0, x1 in [-1, 1] at once, in packed half precision.
//
// The magnitude levels c_0 = 0 < c_1 < ... < c_7 = 1 have growing gaps, so the map F that sends c_j to j and is
// linear in between is concave: F(a) = min_j (S_j * a + j - c_j * S_j) with S_j = 1 / (c_{j+1} - c_j).  Choosing the
// upper neighbour with probability (a - c_j)/(c_{j+1} - c_j) is then the same as rounding F(a) - 0.5 + u to the
// nearest integer for u uniform in (0, 1) (u = 0.5: round to nearest code).  Seven fused multiply-adds and six
// minima serve two elements; the -0.5 is folded into the intercepts.  The integer rounding and the sign are one
// more multiply-add: 1543 +- w lies in [1024, 2048), where half precision has a spacing of one, and 1543 = 0x607
// ends in 7, so the low four bits of the result are the code 7 +- j.  ops/formats.py::nf4_encode_unit computes the
// same numbers step by step (it is the oracle of this function), over every half-precision magnitude.
// rbits: random bits of x0 in the low half and of x1 in the high half (the low 10 bits of each are used).
// Returns code(x0) in bits 0-3 and code(x1) in bits 16-19.
__device__ __forceinline__ uint32_t nf4_encode_pair(float x0, float x1, uint32_t rbits, bool stochastic) {
    constexpr uint16_t kS[7] = {0x497d, 0x4956, 0x4905, 0x4886, 0x47ae, 0x45d8, 0x4295};   // slopes S_j
    constexpr uint16_t kB[7] = {0xb800, 0xb78e, 0xb5b0, 0xacb8, 0x3779, 0x3db9, 0x426b};   // j - c_j * S_j - 0.5
    auto h2 = [](uint32_t bits) { __half2 h; *reinterpret_cast<uint32_t*>(&h) = bits; return h; };
    auto dup = [](uint16_t v) { return static_cast<uint32_t>(v) * 0x00010001u; };
    const __half2 xh = __floats2half2_rn(x0, x1);
    const uint32_t xb = *reinterpret_cast<const uint32_t*>(&xh);
    const __half2 ah = __hmin2(h2(xb & 0x7FFF7FFFu), h2(0x3C003C00u));                        // min(|x|, 1)
    __half2 f = __hfma2(ah, h2(dup(kS[0])), h2(dup(kB[0])));
#pragma unroll
    for (int j = 1; j < 7; ++j) f = __hmin2(f, __hfma2(ah, h2(dup(kS[j])), h2(dup(kB[j]))));
    const __half2 u = stochastic ? __hsub2(h2(0x3C003C00u | (rbits & 0x03FF03FFu)), h2(0x3BFF3BFFu))   // (2r + 1) / 2048
                                 : h2(0x38003800u);                                                    // 0.5
    const __half2 w = __hadd2(f, u);
    const __half2 sgn = h2((xb & 0x80008000u) | 0x3C003C00u);                                  // +-1
    const __half2 code = __hfma2(sgn, w, h2(0x66076607u));                                     // 1543 +- w -> integer
    return *reinterpret_cast<const uint32_t*>(&code) & 0x000F000Fu;
}

// log-uint8 code of v given 1/scale; noise in [-0.5, 0.5) or 0.
__device__ __forceinline__ uint32_t logv_encode(float v, float inv_scale, float noise) {
    if (!(v > 0.0f)) return 0u;
    const float r = fmaxf(v * inv_scale, 5.9604644775390625e-08f);  // 2^-24
    float lg;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(lg) : "f"(r));   // r is a normal number in [2^-24, 1]
    const float pos = fmaf(lg, 10.583333333333334f, 255.0f);
    float q = floorf((pos + 0.5f) + noise);
    q = fminf(fmaxf(q, 1.0f), 255.0f);
    return static_cast<uint32_t>(q);
}

}  // namespace apexb
