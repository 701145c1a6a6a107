// Fused epilogue of the tensor-core GEMMs: one 32-column chunk of an accumulator row, held in
// registers by the thread that owns the row, goes through bias / activation / gated product /
// residual and is stored as fp32 or as a split pair for the next GEMM.
#pragma once
#include "common.cuh"
#include "split.cuh"

#include <cuda.h>

namespace ncmb {

struct TcEpi {
    const float *bias; const float *res; int64_t ldres;
    float *y; float *y_lo; int64_t ldy;
    int y_fmt;                                          // SPLIT_TF32 / SPLIT_H16 when y_lo is set
    int64_t M; int N; int act; int glu;
    const float *colnorm; unsigned long long *best;     // nearest-row mode
    int *err;
    int tma_store;                                      // fp32 result tiles leave through shared memory and TMA stores
    // per-head RMSNorm + rotary embedding of a fused QKV projection (head dim 64), see GemmArgs
    int qk_heads, qk_H;
    const float *qk_qw, *qk_kw, *qk_cos, *qk_sin;
    const int *qk_pos;
    // fp16-pair engine: the activation pair carries a factor 16 and the weight pair was formed from W * 2^e (e per
    // matrix); the accumulator is multiplied by acc_scale = 2^-(4 + e) (exact)
    float acc_scale;
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
// rp: the chunk's eight residual float4 already in registers (only honoured on the vector path, whose
// conditions tc_residual_prefetchable() restates), or null to load them here.
__device__ __forceinline__ bool tc_residual_prefetchable(const TcEpi &ep, int64_t m, int n0, int c0) {
    return ep.res && !ep.glu && m < ep.M && (n0 + c0 + 32 <= ep.N) && ((ep.ldy & 3) == 0) && ((ep.ldres & 3) == 0);
}
__device__ __forceinline__ void tc_epilogue_chunk(const TcEpi &ep, const uint32_t *r, int64_t m, int n0, int c0,
                                                  const float4 *rp = nullptr) {
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
            if (ep.act != ACT_NONE) { v.x = tc_act(v.x, ep.act); v.y = tc_act(v.y, ep.act); v.z = tc_act(v.z, ep.act); v.w = tc_act(v.w, ep.act); }
            if (rr) { float4 q4 = rp ? rp[j >> 2] : *(const float4 *)(rr + j); v.x += q4.x; v.y += q4.y; v.z += q4.z; v.w += q4.w; }
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



// The gated MLP's up-projection in fp16-pair mode, specialised: 32 accumulator columns (interleaved
// gate / up) become 16 outputs silu(gate) * up, each stored as an fp16 pair. SiLU goes through
// ex2.approx / rcp.approx: its few-ulp error is below the 22 significant bits the pair keeps.
// Ragged edges fall back to the generic chunk.
__device__ __forceinline__ bool tc_glu_silu_h16(const TcEpi &ep) {
    return ep.glu && ep.act == ACT_SILU && ep.y_lo && ep.y_fmt == SPLIT_H16 && (ep.ldy & 7) == 0;
}
__device__ __forceinline__ void tc_epilogue_glu_silu_h16(const TcEpi &ep, const uint32_t *r, int64_t m, int n0, int c0) {
    if (m >= ep.M) return;
    if (n0 + c0 + 32 > ep.N) { tc_epilogue_chunk(ep, r, m, n0, c0); return; }
    uint32_t p1[8], p2[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {                       // two outputs (four accumulator columns) per step
        float g0 = __uint_as_float(r[4 * j]), u0 = __uint_as_float(r[4 * j + 1]);
        float g1 = __uint_as_float(r[4 * j + 2]), u1 = __uint_as_float(r[4 * j + 3]);
        if (ep.bias) {
            const float4 b = *(const float4 *)(ep.bias + n0 + c0 + 4 * j);
            g0 += b.x; u0 += b.y; g1 += b.z; u1 += b.w;
        }
        const float o0 = __fmul_rn(__fdividef(g0, 1.0f + __expf(-g0)), u0);
        const float o1 = __fmul_rn(__fdividef(g1, 1.0f + __expf(-g1)), u1);
        h16_pair2(o0, o1, p1[j], p2[j]);
    }
    const int64_t e0 = m * ep.ldy + ((n0 + c0) >> 1);   // first output element; a multiple of 8 halfs (16 bytes)
    uint4 *d1 = (uint4 *)((unsigned short *)ep.y + e0), *d2 = (uint4 *)((unsigned short *)ep.y_lo + e0);
    d1[0] = make_uint4(p1[0], p1[1], p1[2], p1[3]); d1[1] = make_uint4(p1[4], p1[5], p1[6], p1[7]);
    d2[0] = make_uint4(p2[0], p2[1], p2[2], p2[3]); d2[1] = make_uint4(p2[4], p2[5], p2[6], p2[7]);
}

// fp32 result chunk (32 rows of one warp x 32 columns) through shared memory and one TMA store: each
// thread writes its row's eight float4 into a 4 KB staging buffer in the 128-byte-swizzle layout, the
// TMA unit then writes 32 full 128-byte rows (and clips rows >= M itself). A thread-per-row store
// straight to global memory would issue 32 separate 16-byte pieces per instruction.
// Only for chunks that lie fully inside N; `stage` must be 1024-byte aligned.
__device__ __forceinline__ void tc_epilogue_chunk_tma(const TcEpi &ep, const uint32_t *r, int64_t m, int64_t m_warp0, int n0, int c0,
                                                      const float4 *rp, unsigned char *stage, const CUtensorMap *tmY, int lane) {
    // the previous store out of this buffer must have finished reading it
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
    const float *rr = (ep.res && m < ep.M) ? ep.res + m * ep.ldres + n0 + c0 : nullptr;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        if (ep.bias) {
            float4 b = *(const float4 *)(ep.bias + n0 + c0 + j);
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        }
        if (ep.act != ACT_NONE) { v.x = tc_act(v.x, ep.act); v.y = tc_act(v.y, ep.act); v.z = tc_act(v.z, ep.act); v.w = tc_act(v.w, ep.act); }
        if (rr) { float4 q4 = rp ? rp[j >> 2] : *(const float4 *)(rr + j); v.x += q4.x; v.y += q4.y; v.z += q4.z; v.w += q4.w; }
        *(float4 *)(stage + lane * 128 + ((((j >> 2) ^ (lane & 7)) & 7) << 4)) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                     ::"l"(tmY), "r"(n0 + c0), "r"((int)m_warp0), "r"((uint32_t)__cvta_generic_to_shared(stage)) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
}

// fp32 tile out through staging + TMA store, with the residual arriving the coalesced way: the warp fetched the
// chunk's 32 x 32 residual block together (lane L, step i: row 4 i + L / 8, four columns at 4 (L % 8): full 128-byte
// row segments per request, where a thread reading its own row touches 32 separate sectors per request) and holds it
// in `coop`; here the block goes through the swizzled staging buffer, each thread adds its row to its accumulators in
// place, and the buffer leaves by TMA store.
__device__ __forceinline__ void tc_epilogue_chunk_tma_coop(const TcEpi &ep, const uint32_t *r, int64_t m_warp0, int n0, int c0,
                                                           const float4 *coop, unsigned char *stage, const CUtensorMap *tmY, int lane) {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");    // the previous store has read the buffer
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int row = i * 4 + (lane >> 3), c4 = lane & 7;
        *(float4 *)(stage + row * 128 + (((c4 ^ (row & 7)) & 7) << 4)) = coop[i];
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        if (ep.bias) {
            float4 b = *(const float4 *)(ep.bias + n0 + c0 + j);
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        }
        if (ep.act != ACT_NONE) { v.x = tc_act(v.x, ep.act); v.y = tc_act(v.y, ep.act); v.z = tc_act(v.z, ep.act); v.w = tc_act(v.w, ep.act); }
        float4 *slot = (float4 *)(stage + lane * 128 + ((((j >> 2) ^ (lane & 7)) & 7) << 4));
        const float4 q4 = *slot;
        v.x += q4.x; v.y += q4.y; v.z += q4.z; v.w += q4.w;
        *slot = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                     ::"l"(tmY), "r"(n0 + c0), "r"((int)m_warp0), "r"((uint32_t)__cvta_generic_to_shared(stage)) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
}

// One head (64 columns starting at n0) of row m of a fused QKV projection: bias, then for query / key heads the
// per-head RMSNorm (x * rsqrt(mean x^2 + 1e-6) * w, the products rounded one by one) and the rotation of the pairs
// (d, d + 32) with the table row of the token's position -- the arithmetic of qk_post(), on values that are still
// in registers. r0 / r1 hold columns [0, 32) / [32, 64) of the head. Both halves then leave through the warp's
// staging buffer and two TMA stores.
__device__ __forceinline__ void tc_epilogue_head_qkpost(const TcEpi &ep, uint32_t *r0, uint32_t *r1, int64_t m, int64_t m_warp0,
                                                       int n0, unsigned char *stage, const CUtensorMap *tmY, int lane) {
    const int head = n0 >> 6;
    if (ep.bias) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 b0 = *(const float4 *)(ep.bias + n0 + j), b1 = *(const float4 *)(ep.bias + n0 + 32 + j);
            r0[j] = __float_as_uint(__uint_as_float(r0[j]) + b0.x); r0[j + 1] = __float_as_uint(__uint_as_float(r0[j + 1]) + b0.y);
            r0[j + 2] = __float_as_uint(__uint_as_float(r0[j + 2]) + b0.z); r0[j + 3] = __float_as_uint(__uint_as_float(r0[j + 3]) + b0.w);
            r1[j] = __float_as_uint(__uint_as_float(r1[j]) + b1.x); r1[j + 1] = __float_as_uint(__uint_as_float(r1[j + 1]) + b1.y);
            r1[j + 2] = __float_as_uint(__uint_as_float(r1[j + 2]) + b1.z); r1[j + 3] = __float_as_uint(__uint_as_float(r1[j + 3]) + b1.w);
        }
    }
    if (head < ep.qk_heads && m < ep.M) {
        const float *nw = head < ep.qk_H ? ep.qk_qw : ep.qk_kw;
        if (nw) {
            float s[32];                                   // pair sums, added up in the order of a 32-lane butterfly
#pragma unroll
            for (int i = 0; i < 32; i++) { const float a = __uint_as_float(r0[i]), b = __uint_as_float(r1[i]); s[i] = a * a + b * b; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int i = 0; i < o; i++) s[i] += s[i + o];
            const float rinv = 1.0f / sqrtf(s[0] / 64.0f + 1e-6f);
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 w0 = *(const float4 *)(nw + j), w1 = *(const float4 *)(nw + 32 + j);
                r0[j] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r0[j]), rinv), w0.x));
                r0[j + 1] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r0[j + 1]), rinv), w0.y));
                r0[j + 2] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r0[j + 2]), rinv), w0.z));
                r0[j + 3] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r0[j + 3]), rinv), w0.w));
                r1[j] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r1[j]), rinv), w1.x));
                r1[j + 1] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r1[j + 1]), rinv), w1.y));
                r1[j + 2] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r1[j + 2]), rinv), w1.z));
                r1[j + 3] = __float_as_uint(__fmul_rn(__fmul_rn(__uint_as_float(r1[j + 3]), rinv), w1.w));
            }
        }
        if (ep.qk_cos) {
            const float *cs = ep.qk_cos + (int64_t)ep.qk_pos[m] * 64, *sn = ep.qk_sin + (int64_t)ep.qk_pos[m] * 64;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const float4 c0 = *(const float4 *)(cs + j), c1 = *(const float4 *)(cs + 32 + j);
                const float4 s0 = *(const float4 *)(sn + j), s1 = *(const float4 *)(sn + 32 + j);
                const float cc0[4] = {c0.x, c0.y, c0.z, c0.w}, cc1[4] = {c1.x, c1.y, c1.z, c1.w};
                const float ss0[4] = {s0.x, s0.y, s0.z, s0.w}, ss1[4] = {s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float x0 = __uint_as_float(r0[j + e]), x1 = __uint_as_float(r1[j + e]);
                    r0[j + e] = __float_as_uint(__fadd_rn(__fmul_rn(x0, cc0[e]), __fmul_rn(-x1, ss0[e])));
                    r1[j + e] = __float_as_uint(__fadd_rn(__fmul_rn(x1, cc1[e]), __fmul_rn(x0, ss1[e])));
                }
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const uint32_t *r = half ? r1 : r0;
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous store has read the buffer
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            *(float4 *)(stage + lane * 128 + ((((j >> 2) ^ (lane & 7)) & 7) << 4)) =
                make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                         ::"l"(tmY), "r"(n0 + half * 32), "r"((int)m_warp0), "r"((uint32_t)__cvta_generic_to_shared(stage)) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
}

} // namespace ncmb
