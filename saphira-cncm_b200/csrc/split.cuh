// Split pairs: how a kernel that produces the input of a tensor-core GEMM writes it so the GEMM
// can consume fp32-grade operands without a separate conversion pass.
//   SPLIT_TF32  y = rn_tf32(v), y_lo = v - y (both float arrays; three TF32 MMAs recover the product)
//   SPLIT_H16   y, y_lo are read as __half arrays with the SAME element stride: with t = 16 v,
//               y = rn_f16(t) and y_lo = rn_f16(t - y). The remainder is NOT scaled, so the GEMM adds
//               x1 W1 + x1 W2 + x2 W1 in ONE accumulator; the fixed factor 16 keeps remainders of values
//               down to |v| = 2^-7 in the normal fp16 range (below that they are exact to 2^-29 absolute,
//               which against K-term sums of such values is the fp32 rounding level). The GEMM's epilogue
//               divides the factor out. Values beyond +-4094 saturate.
#pragma once
#include <cuda_fp16.h>

namespace ncmb {

constexpr float H16_X_SCALE = 16.0f, H16_X_UNSCALE = 1.0f / 16.0f;

__device__ __forceinline__ float split_tf32_hi(float v) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
    return __uint_as_float(u);
}
__device__ __forceinline__ unsigned short f16_sat(float v) {
    unsigned short h;
    asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(h) : "f"(v));
    return h;
}
__device__ __forceinline__ void h16_pair(float v, unsigned short &hi, unsigned short &lo) {
    const float t = v * H16_X_SCALE;
    hi = f16_sat(t);
    lo = f16_sat(t - __half2float(__ushort_as_half(hi)));
}
// two values at once, packed (a in the low half-word), without the format's factor: hi = rn_f16(v),
// lo = rn_f16((v - hi) * lo_scale); one conversion instruction per packed result instead of one per value
__device__ __forceinline__ void h16_pair2_raw(float a, float b, uint32_t &hi, uint32_t &lo, float lo_scale) {
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(b), "f"(a));
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"((b - f.y) * lo_scale), "f"((a - f.x) * lo_scale));
}
// the SPLIT_H16 pair of two values, packed: the same roundings as h16_pair
__device__ __forceinline__ void h16_pair2(float a, float b, uint32_t &hi, uint32_t &lo) {
    h16_pair2_raw(a * H16_X_SCALE, b * H16_X_SCALE, hi, lo, 1.0f);
}
// element index i into both arrays
__device__ __forceinline__ void store_split1(float *y, float *y_lo, int64_t i, float v, int fmt) {
    if (fmt == SPLIT_H16) {
        unsigned short hi, lo;
        h16_pair(v, hi, lo);
        ((unsigned short *)y)[i] = hi; ((unsigned short *)y_lo)[i] = lo;
    } else {
        float hi = split_tf32_hi(v);
        y[i] = hi; y_lo[i] = v - hi;
    }
}
// four consecutive elements, i a multiple of 4 and both rows 16-byte aligned
__device__ __forceinline__ void store_split4(float *y, float *y_lo, int64_t i, float4 v, int fmt) {
    if (fmt == SPLIT_H16) {
        uint32_t h0, h1, l0, l1;
        h16_pair2(v.x, v.y, h0, l0); h16_pair2(v.z, v.w, h1, l1);
        *(uint2 *)((unsigned short *)y + i) = make_uint2(h0, h1);
        *(uint2 *)((unsigned short *)y_lo + i) = make_uint2(l0, l1);
    } else {
        float4 h = make_float4(split_tf32_hi(v.x), split_tf32_hi(v.y), split_tf32_hi(v.z), split_tf32_hi(v.w));
        *(float4 *)(y + i) = h;
        *(float4 *)(y_lo + i) = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
    }
}

} // namespace ncmb
