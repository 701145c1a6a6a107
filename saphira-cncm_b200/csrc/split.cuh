// Split pairs: how a kernel that produces the input of a tensor-core GEMM writes it so the GEMM
// can consume fp32-grade operands without a separate conversion pass.
//   SPLIT_TF32  y = rn_tf32(v), y_lo = v - y (both float arrays; three TF32 MMAs recover the product)
//   SPLIT_H16   y, y_lo are read as __half arrays with the SAME element stride: y = rn_f16(v) and
//               y_lo = rn_f16((v - y) * 2^11); the GEMM accumulates the cross terms separately and
//               scales them back by 2^-11. Values beyond the fp16 range saturate to +-65504.
#pragma once
#include <cuda_fp16.h>

namespace ncmb {

constexpr float H16_LO_SCALE = 2048.0f, H16_LO_UNSCALE = 1.0f / 2048.0f;

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
    hi = f16_sat(v);
    lo = f16_sat((v - __half2float(__ushort_as_half(hi))) * H16_LO_SCALE);
}
// two values at once, packed (a in the low half-word): the same roundings as h16_pair, with one conversion
// instruction per packed result instead of one per value
__device__ __forceinline__ void h16_pair2(float a, float b, uint32_t &hi, uint32_t &lo, float lo_scale = H16_LO_SCALE) {
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(b), "f"(a));
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"((b - f.y) * lo_scale), "f"((a - f.x) * lo_scale));
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
