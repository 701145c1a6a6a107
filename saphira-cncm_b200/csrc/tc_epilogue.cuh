// Fused epilogue of the tensor-core GEMMs: one 32-column chunk of an accumulator row, held in
// registers by the thread that owns the row, goes through bias / activation / gated product /
// residual and is stored as fp32 or as a split pair for the next GEMM.
#pragma once
#include "common.cuh"
#include "split.cuh"

namespace ncmb {

struct TcEpi {
    const float *bias; const float *res; int64_t ldres;
    float *y; float *y_lo; int64_t ldy;
    int y_fmt;                                          // SPLIT_TF32 / SPLIT_H16 when y_lo is set
    int64_t M; int N; int act; int glu;
    const float *colnorm; unsigned long long *best;     // nearest-row mode
    int *err;
};


__device__ __forceinline__ float tc_act(float v, int act) {
    switch (act) {
        case ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.7071067811865475f));
        case ACT_GELU_TANH: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case ACT_SILU: return v / (1.0f + expf(-v));
        case ACT_RELU2: { float r = v > 0.f ? v : 0.f; return r * r; }
        default: return v;
    }
}

// Fused epilogue for one 32-column chunk of an accumulator row held in registers.
__device__ __forceinline__ void tc_epilogue_chunk(const TcEpi &ep, const uint32_t *r, int64_t m, int n0, int c0) {
    if (m >= ep.M || n0 + c0 >= ep.N) return;
    if (ep.glu) {
        // interleaved gate/up columns: out[j] = act(acc[2j] + b[2j]) * (acc[2j+1] + b[2j+1])
        float *yr = ep.y + m * ep.ldy + ((n0 + c0) >> 1);
        float *lr = ep.y_lo ? ep.y_lo + m * ep.ldy + ((n0 + c0) >> 1) : nullptr;
        const bool full = (n0 + c0 + 32 <= ep.N) && ((ep.ldy & 3) == 0);
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int n = n0 + c0 + 2 * (j + e);
                float g = __uint_as_float(r[2 * (j + e)]), u = __uint_as_float(r[2 * (j + e) + 1]);
                if (ep.bias && n + 1 < ep.N) { g += ep.bias[n]; u += ep.bias[n + 1]; }
                o[e] = __fmul_rn(tc_act(g, ep.act), u);
            }
            if (full) {
                float4 v = make_float4(o[0], o[1], o[2], o[3]);
                if (lr) store_split4(ep.y, ep.y_lo, m * ep.ldy + ((n0 + c0) >> 1) + j, v, ep.y_fmt);
                else *(float4 *)(yr + j) = v;
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    int n = n0 + c0 + 2 * (j + e);
                    if (n + 1 < ep.N) {
                        if (lr) store_split1(ep.y, ep.y_lo, m * ep.ldy + ((n0 + c0) >> 1) + j + e, o[e], ep.y_fmt);
                        else yr[j + e] = o[e];
                    }
                }
            }
        }
        return;
    }
    float *yr = ep.y + m * ep.ldy + n0 + c0;
    const float *rr = ep.res ? ep.res + m * ep.ldres + n0 + c0 : nullptr;
    const bool full = (n0 + c0 + 32 <= ep.N) && ((ep.ldy & 3) == 0) && (!rr || (ep.ldres & 3) == 0);
    if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            if (ep.bias) {
                float4 b = *(const float4 *)(ep.bias + n0 + c0 + j);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            v.x = tc_act(v.x, ep.act); v.y = tc_act(v.y, ep.act); v.z = tc_act(v.z, ep.act); v.w = tc_act(v.w, ep.act);
            if (rr) { float4 q4 = *(const float4 *)(rr + j); v.x += q4.x; v.y += q4.y; v.z += q4.z; v.w += q4.w; }
            if (ep.y_lo) store_split4(ep.y, ep.y_lo, m * ep.ldy + n0 + c0 + j, v, ep.y_fmt);
            else *(float4 *)(yr + j) = v;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++) {
            int n = n0 + c0 + j;
            if (n < ep.N) {
                float v = __uint_as_float(r[j]);
                if (ep.bias) v += ep.bias[n];
                v = tc_act(v, ep.act);
                if (rr) v += rr[j];
                if (ep.y_lo) store_split1(ep.y, ep.y_lo, m * ep.ldy + n, v, ep.y_fmt);
                else yr[j] = v;
            }
        }
    }
}



} // namespace ncmb
