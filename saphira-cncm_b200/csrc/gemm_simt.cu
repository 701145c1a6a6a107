// fp32 CUDA-core GEMM: y = act(x W^T + bias) (+ res), both operands K-major.
// This is the exact-arithmetic engine (fp32 FMA accumulation): it serves shapes the
// tensor-core engine does not take (tiny M, odd K) and gemm mode 0, and it is what
// linear_fwd of the reference kernel API (src/ncm.h:146) maps to in that mode.
#include "common.cuh"

namespace ncmb {

__device__ __forceinline__ float act_fn(float v, int act) {
    switch (act) {
        case ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.7071067811865475f));
        case ACT_GELU_TANH: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case ACT_SILU: return v / (1.0f + expf(-v));
        case ACT_RELU2: { float r = v > 0.f ? v : 0.f; return r * r; }
        default: return v;
    }
}

struct GemmDev {
    const float *x; int64_t ldx;
    const float *W;
    const float *bias;
    const float *res; int64_t ldres;
    float *y; int64_t ldy;
    int64_t M; int N, K;
    int act;
    int vec;        // 1: K % 4 == 0 and x / W rows are 16-byte aligned
    int ln_kind; const float *ln_w, *ln_b; float ln_eps;
    float *y2; int y2_col0; int64_t ldy2; const int *y2_step_d; int64_t y2_step;
    const unsigned short *W16;      // optional exact bf16 copy of W (GEMV kernel only): half the bytes to stream
};

// ---- tiled kernel: BM x BN output tile per CTA, BK-deep stages, TMxTN per thread ----
// Each thread owns two 4-wide column groups (tx*4 and BN/2 + tx*4) and two 4-high row
// groups, so shared-memory reads are conflict-free float4s.
template <int BM, int BN, int BK>
__global__ void __launch_bounds__((BM / 8) * (BN / 8)) k_gemm_tiled(GemmDev a) {
    constexpr int NT = (BM / 8) * (BN / 8);
    constexpr int LDA = BM + 4, LDB = BN + 4;
    __shared__ __align__(16) float As[2][BK][LDA];
    __shared__ __align__(16) float Bs[2][BK][LDB];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / 8), ty = tid / (BN / 8);
    const int64_t m0 = (int64_t)blockIdx.y * BM;
    const int n0 = blockIdx.x * BN;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

    constexpr int KQ = BK / 4;                    // float4 per tile row
    constexpr int A_ITERS = (BM * KQ + NT - 1) / NT;
    constexpr int B_ITERS = (BN * KQ + NT - 1) / NT;
    float4 ra[A_ITERS], rb[B_ITERS];

    auto gload = [&](int k0) {
#pragma unroll
        for (int it = 0; it < A_ITERS; it++) {
            int i = tid + it * NT;
            int row = i / KQ, kq = i % KQ;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            int64_t m = m0 + row;
            int k = k0 + kq * 4;
            if (i < BM * KQ && m < a.M) {
                const float *p = a.x + m * a.ldx + k;
                if (a.vec && k + 3 < a.K) v = *(const float4 *)p;
                else {
                    if (k < a.K) v.x = p[0];
                    if (k + 1 < a.K) v.y = p[1];
                    if (k + 2 < a.K) v.z = p[2];
                    if (k + 3 < a.K) v.w = p[3];
                }
            }
            ra[it] = v;
        }
#pragma unroll
        for (int it = 0; it < B_ITERS; it++) {
            int i = tid + it * NT;
            int row = i / KQ, kq = i % KQ;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            int n = n0 + row;
            int k = k0 + kq * 4;
            if (i < BN * KQ && n < a.N) {
                const float *p = a.W + (int64_t)n * a.K + k;
                if (a.vec && k + 3 < a.K) v = *(const float4 *)p;
                else {
                    if (k < a.K) v.x = p[0];
                    if (k + 1 < a.K) v.y = p[1];
                    if (k + 2 < a.K) v.z = p[2];
                    if (k + 3 < a.K) v.w = p[3];
                }
            }
            rb[it] = v;
        }
    };
    auto sstore = [&](int buf) {
#pragma unroll
        for (int it = 0; it < A_ITERS; it++) {
            int i = tid + it * NT;
            if (i < BM * KQ) {
                int row = i / KQ, kq = i % KQ;
                As[buf][kq * 4 + 0][row] = ra[it].x; As[buf][kq * 4 + 1][row] = ra[it].y;
                As[buf][kq * 4 + 2][row] = ra[it].z; As[buf][kq * 4 + 3][row] = ra[it].w;
            }
        }
#pragma unroll
        for (int it = 0; it < B_ITERS; it++) {
            int i = tid + it * NT;
            if (i < BN * KQ) {
                int row = i / KQ, kq = i % KQ;
                Bs[buf][kq * 4 + 0][row] = rb[it].x; Bs[buf][kq * 4 + 1][row] = rb[it].y;
                Bs[buf][kq * 4 + 2][row] = rb[it].z; Bs[buf][kq * 4 + 3][row] = rb[it].w;
            }
        }
    };

    const int nk = (a.K + BK - 1) / BK;
    gload(0);
    sstore(0);
    __syncthreads();
    for (int kt = 0; kt < nk; kt++) {
        int buf = kt & 1;
        if (kt + 1 < nk) gload((kt + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float4 a0 = *(const float4 *)&As[buf][k][ty * 4];
            float4 a1 = *(const float4 *)&As[buf][k][BM / 2 + ty * 4];
            float4 b0 = *(const float4 *)&Bs[buf][k][tx * 4];
            float4 b1 = *(const float4 *)&Bs[buf][k][BN / 2 + tx * 4];
            float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (kt + 1 < nk) sstore(buf ^ 1);
        __syncthreads();
    }
    // epilogue
#pragma unroll
    for (int i = 0; i < 8; i++) {
        int64_t m = m0 + (i < 4 ? ty * 4 + i : BM / 2 + ty * 4 + (i - 4));
        if (m >= a.M) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            int n = n0 + (j < 4 ? tx * 4 + j : BN / 2 + tx * 4 + (j - 4));
            if (n >= a.N) continue;
            float v = acc[i][j];
            if (a.bias) v += a.bias[n];
            v = act_fn(v, a.act);
            if (a.res) v += a.res[m * a.ldres + n];
            a.y[m * a.ldy + n] = v;
        }
    }
}

// ---- skinny kernel (M small): one warp per output column, the weight row is streamed
// once with 128-bit loads and reused for up to MT activation rows held in registers. ----
template <int MT>
__global__ void __launch_bounds__(256) k_gemm_skinny(GemmDev a) {
    int warp = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    int lane = threadIdx.x & 31;
    if (warp >= a.N) return;
    const float *wr = a.W + (int64_t)warp * a.K;
    for (int64_t mb = 0; mb < a.M; mb += MT) {
        float acc[MT];
#pragma unroll
        for (int i = 0; i < MT; i++) acc[i] = 0.f;
        if (a.vec) {
            for (int k = lane * 4; k < a.K; k += 128) {
                float4 w = *(const float4 *)(wr + k);
#pragma unroll
                for (int i = 0; i < MT; i++) {
                    if (mb + i < a.M) {
                        float4 xv = *(const float4 *)(a.x + (mb + i) * a.ldx + k);
                        acc[i] = fmaf(xv.x, w.x, acc[i]); acc[i] = fmaf(xv.y, w.y, acc[i]);
                        acc[i] = fmaf(xv.z, w.z, acc[i]); acc[i] = fmaf(xv.w, w.w, acc[i]);
                    }
                }
            }
        } else {
            for (int k = lane; k < a.K; k += 32) {
                float w = wr[k];
#pragma unroll
                for (int i = 0; i < MT; i++)
                    if (mb + i < a.M) acc[i] = fmaf(a.x[(mb + i) * a.ldx + k], w, acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < MT; i++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < MT; i++) {
                int64_t m = mb + i;
                if (m < a.M) {
                    float v = acc[i];
                    if (a.bias) v += a.bias[warp];
                    v = act_fn(v, a.act);
                    if (a.res) v += a.res[m * a.ldres + warp];
                    a.y[m * a.ldy + warp] = v;
                }
            }
        }
    }
}

// ---- GEMV-like kernel (M <= 8 rows per pass, vector path): one CTA per GV_NC output columns, all 256 threads
// stride over K together, so every thread has its 128-bit weight loads of all columns in flight at once
// (the weights are read exactly once, coalesced 512 bytes per warp and column); partial dot products are
// reduced by warp shuffles and one shared-memory pass. Decode steps (one token per sequence) live here: they
// are bound by streaming the weights, not by arithmetic.
// The kernel is launched with programmatic stream serialization: it lets its successor start at once
// (griddepcontrol.launch_dependents), requests the weights of its first GV_PF k-steps -- which no kernel of a
// decode step writes -- and only then waits for its predecessor (griddepcontrol.wait) before touching x. So
// the launch latency and the DRAM latency of the weight stream run under the previous kernel. ----
// four consecutive weights of row `row` at column k: fp32, or bf16 widened exactly (bits << 16)
__device__ __forceinline__ float4 gv_w4(const GemmDev &a, int64_t row, int k) {
    if (a.W16) {
        const uint2 u = __ldg((const uint2 *)(a.W16 + row * a.K + k));
        return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                           __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
    }
    return __ldg((const float4 *)(a.W + row * a.K + k));
}

template <int MT, int GV_NC, int GV_PF>
__global__ void __launch_bounds__(256) k_gemv(GemmDev a) {
    __shared__ float red[8][MT][GV_NC];
    __shared__ float stat[8][MT], s_mean[MT], s_rstd[MT];
    const int n0 = blockIdx.x * GV_NC;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    int64_t wr[GV_NC];                                   // weight rows of this CTA's columns
#pragma unroll
    for (int c = 0; c < GV_NC; c++) wr[c] = min(n0 + c, a.N - 1);
    float4 wpre[GV_PF][GV_NC];
#pragma unroll
    for (int p = 0; p < GV_PF; p++) {
        const int k = tid * 4 + p * 1024;
        if (k < a.K) {
#pragma unroll
            for (int c = 0; c < GV_NC; c++) wpre[p][c] = gv_w4(a, wr[c], k);
        }
    }
    pdl_wait();
    for (int64_t mb = 0; mb < a.M; mb += MT) {
        float acc[MT][GV_NC];
#pragma unroll
        for (int i = 0; i < MT; i++)
#pragma unroll
            for (int c = 0; c < GV_NC; c++) acc[i][c] = 0.f;
        if (a.ln_kind) {
            // row statistics of the MT input rows (every CTA repeats them: a row is a few KB out of L2)
            float mean[MT];
            for (int pass = 0; pass < 2; pass++) {
                if (pass == 0 && a.ln_kind == 2) {
#pragma unroll
                    for (int i = 0; i < MT; i++) mean[i] = 0.f;
                    continue;                                   // RMSNorm: no mean
                }
                float part[MT];
#pragma unroll
                for (int i = 0; i < MT; i++) part[i] = 0.f;
                for (int k = tid * 4; k < a.K; k += 1024) {
#pragma unroll
                    for (int i = 0; i < MT; i++) {
                        if (mb + i < a.M) {
                            const float4 v = *(const float4 *)(a.x + (mb + i) * a.ldx + k);
                            if (pass == 0) part[i] += (v.x + v.y) + (v.z + v.w);
                            else {
                                float d0 = v.x - mean[i], d1 = v.y - mean[i], d2 = v.z - mean[i], d3 = v.w - mean[i];
                                part[i] += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
                            }
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < MT; i++) {
                    float v = part[i];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == 0) stat[warp][i] = v;
                }
                __syncthreads();
                if (tid < MT) {
                    float v = 0.f;
#pragma unroll
                    for (int w8 = 0; w8 < 8; w8++) v += stat[w8][tid];
                    v /= (float)a.K;
                    if (pass == 0) s_mean[tid] = v; else s_rstd[tid] = 1.0f / sqrtf(v + a.ln_eps);
                }
                __syncthreads();
                if (pass == 0) {
#pragma unroll
                    for (int i = 0; i < MT; i++) mean[i] = s_mean[i];
                }
            }
        }
        auto kstep = [&](int k, const float4 *w) {
            float4 lw = make_float4(1.f, 1.f, 1.f, 1.f), lb = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.ln_kind) {
                if (a.ln_w) lw = __ldg((const float4 *)(a.ln_w + k));
                if (a.ln_b) lb = __ldg((const float4 *)(a.ln_b + k));
            }
#pragma unroll
            for (int i = 0; i < MT; i++) {
                if (mb + i < a.M) {
                    float4 xv = *(const float4 *)(a.x + (mb + i) * a.ldx + k);
                    if (a.ln_kind) {   // unfused mul / mul / add like the stand-alone norm kernels
                        const float mu = a.ln_kind == 1 ? s_mean[i] : 0.f, rs = s_rstd[i];
                        xv.x = __fadd_rn(__fmul_rn(__fmul_rn(xv.x - mu, rs), lw.x), lb.x);
                        xv.y = __fadd_rn(__fmul_rn(__fmul_rn(xv.y - mu, rs), lw.y), lb.y);
                        xv.z = __fadd_rn(__fmul_rn(__fmul_rn(xv.z - mu, rs), lw.z), lb.z);
                        xv.w = __fadd_rn(__fmul_rn(__fmul_rn(xv.w - mu, rs), lw.w), lb.w);
                    }
#pragma unroll
                    for (int c = 0; c < GV_NC; c++) {
                        acc[i][c] = fmaf(xv.x, w[c].x, acc[i][c]); acc[i][c] = fmaf(xv.y, w[c].y, acc[i][c]);
                        acc[i][c] = fmaf(xv.z, w[c].z, acc[i][c]); acc[i][c] = fmaf(xv.w, w[c].w, acc[i][c]);
                    }
                }
            }
        };
#pragma unroll
        for (int p = 0; p < GV_PF; p++) {
            const int k = tid * 4 + p * 1024;
            if (k < a.K) kstep(k, wpre[p]);
        }
        for (int k = tid * 4 + GV_PF * 1024; k < a.K; k += 1024) {
            float4 w[GV_NC];
#pragma unroll
            for (int c = 0; c < GV_NC; c++) w[c] = gv_w4(a, wr[c], k);
            kstep(k, w);
        }
#pragma unroll
        for (int i = 0; i < MT; i++)
#pragma unroll
            for (int c = 0; c < GV_NC; c++) {
                float v = acc[i][c];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) red[warp][i][c] = v;
            }
        __syncthreads();
        if (tid < MT * GV_NC) {
            const int i = tid / GV_NC, c = tid % GV_NC;
            const int64_t m = mb + i; const int n = n0 + c;
            if (m < a.M && n < a.N) {
                float v = 0.f;
#pragma unroll
                for (int w8 = 0; w8 < 8; w8++) v += red[w8][i][c];
                if (a.bias) v += a.bias[n];
                v = act_fn(v, a.act);
                if (a.res) v += a.res[m * a.ldres + n];
                a.y[m * a.ldy + n] = v;
                if (a.y2 && n >= a.y2_col0)
                    a.y2[m * a.ldy2 + (a.y2_step_d ? (int64_t)(*a.y2_step_d) * a.y2_step : 0) + (n - a.y2_col0)] = v;
            }
        }
        __syncthreads();
    }
}

// ---- decode-step GEMV, up to four rows: one WARP per pair of weight rows ----
// A decode step of one to four sequences is a chain of matrix-vector products whose only real cost is streaming
// the weights once. Here a warp owns two weight rows at a time: lane l takes eight consecutive elements of every
// 256-element chunk of K (one 16-byte load of bf16 weights, two of fp32), all loads of up to four chunks of both
// rows are issued before any is used, partial sums are reduced by shuffles alone, and lane 0 finishes the pair --
// so there is no block-wide reduction and no shared-memory traffic per output. The input rows are staged (and
// normalised, when a norm is fused) in shared memory once per CTA; CTAs are persistent over the row pairs. Which
// two rows form a pair is free, and three epilogues use that:
//   plain   rows (2g, 2g + 1)
//   gated   rows (g, half + g) of a [gate ; up] matrix: out[g] = act(gate) * up -- no separate gating pass
//   rotary  rows (h*hd + d, h*hd + d + hd/2) of the query / key heads of a fused QKV projection: the pair is
//           rotated before it is stored, and K|V columns go straight to the cache -- no rotation pass, no copy
// Launched with programmatic stream serialization: the first loads of the first pair are issued before the wait
// for the predecessor (weights are not written by any kernel of a decode step).
struct GemvW {
    const float *x; int64_t ldx;
    const float *W; const unsigned short *W16;
    const float *bias; const float *res; int64_t ldres;
    float *y; int64_t ldy;
    int M, N, K, act;
    int ln_kind; const float *ln_w, *ln_b; float ln_eps;
    float *y2; int y2_col0; int64_t ldy2; const int *y2_step_d; int64_t y2_step;
    int pair_half;
    const float *rope_cos, *rope_sin; const int *rope_pos, *rope_step_d; int64_t rope_pos_step; int rope_cols, hd;
    int ngroups;
    const char *pf; unsigned long long pf_bytes;      // the next kernel's weights, for L2 (null: none)
};

// Each CTA asks L2 for its slice of the NEXT kernel's weight matrix (bulk prefetch, 16-byte granules, up to 32 KB per
// instruction): a hint with no completion to wait for.
__device__ __forceinline__ void gw_prefetch_next(const GemvW &p) {
    if (!p.pf || threadIdx.x != 0) return;
    const unsigned long long share = ((p.pf_bytes + gridDim.x - 1) / gridDim.x + 15ull) & ~15ull;
    unsigned long long off = (unsigned long long)blockIdx.x * share;
    const unsigned long long end = off + share < p.pf_bytes ? off + share : (p.pf_bytes & ~15ull);
    for (; off < end; off += 32768ull) {
        const unsigned n = (unsigned)(end - off < 32768ull ? end - off : 32768ull);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.pf + off), "r"(n) : "memory");
    }
}

constexpr int GW_U = 4;                      // chunks of 256 elements whose loads are in flight together

template <bool W16>
struct GwTile { uint4 a[GW_U], b[GW_U]; };   // fp32 weights: a = elements 0..3, b = elements 4..7 of the lane's eight; bf16: a only

template <bool W16>
__device__ __forceinline__ void gw_load(const GemvW &p, int64_t row, int c0, int lane, GwTile<W16> &t, int cstep = 1) {
#pragma unroll
    for (int u = 0; u < GW_U; u++) {
        const int k = (c0 + u * cstep) * 256 + lane * 8;
        if (k < p.K) {
            if (W16) t.a[u] = __ldg((const uint4 *)(p.W16 + row * p.K + k));
            else {
                t.a[u] = __ldg((const uint4 *)(p.W + row * p.K + k));
                t.b[u] = __ldg((const uint4 *)(p.W + row * p.K + k + 4));
            }
        }
    }
}

template <bool W16>
__device__ __forceinline__ void gw_w8(const GwTile<W16> &t, int u, float *w) {
    if (W16) {
        w[0] = __uint_as_float(t.a[u].x << 16); w[1] = __uint_as_float(t.a[u].x & 0xffff0000u);
        w[2] = __uint_as_float(t.a[u].y << 16); w[3] = __uint_as_float(t.a[u].y & 0xffff0000u);
        w[4] = __uint_as_float(t.a[u].z << 16); w[5] = __uint_as_float(t.a[u].z & 0xffff0000u);
        w[6] = __uint_as_float(t.a[u].w << 16); w[7] = __uint_as_float(t.a[u].w & 0xffff0000u);
    } else {
        w[0] = __uint_as_float(t.a[u].x); w[1] = __uint_as_float(t.a[u].y); w[2] = __uint_as_float(t.a[u].z); w[3] = __uint_as_float(t.a[u].w);
        w[4] = __uint_as_float(t.b[u].x); w[5] = __uint_as_float(t.b[u].y); w[6] = __uint_as_float(t.b[u].z); w[7] = __uint_as_float(t.b[u].w);
    }
}

// the two weight rows of pair g
__device__ __forceinline__ void gw_rows(const GemvW &p, int g, int &r0, int &r1) {
    if (p.pair_half) { r0 = g; r1 = g + p.pair_half; return; }
    const int half = p.hd >> 1, gr = p.rope_cols >> 1;
    if (p.rope_cos && g < gr) { r0 = (g / half) * p.hd + g % half; r1 = r0 + half; return; }
    r0 = p.rope_cols + 2 * (g - (p.rope_cos ? gr : 0));
    if (!p.rope_cos) r0 = 2 * g;
    r1 = r0 + 1;
}

// lane 0 of the warp that holds the finished sums of pair g (rows c_r0, c_r1): bias, the pair's epilogue, stores
template <int MT>
__device__ __forceinline__ void gw_epilogue(const GemvW &p, int g, int c_r0, int c_r1, const float *acc0, const float *acc1) {
    const bool has1 = c_r1 < p.N;
    const float b0 = p.bias ? p.bias[c_r0] : 0.f, b1 = (p.bias && has1) ? p.bias[c_r1] : 0.f;
    const int gr = p.rope_cols >> 1;
    const bool rot = p.rope_cos && !p.pair_half && (g < gr);
#pragma unroll
    for (int m = 0; m < MT; m++) {
        if (m >= p.M) break;
        float v0 = acc0[m] + b0, v1 = acc1[m] + b1;
        if (p.pair_half) {
            p.y[(int64_t)m * p.ldy + g] = act_fn(v0, p.act) * v1;
            continue;
        }
        if (rot) {
            const int half = p.hd >> 1, d = c_r0 % p.hd;
            const int64_t pos = (int64_t)p.rope_pos[(p.rope_step_d ? (int64_t)(*p.rope_step_d) * p.rope_pos_step : 0) + m] * p.hd;
            const float c0v = p.rope_cos[pos + d], c1v = p.rope_cos[pos + d + half], s0v = p.rope_sin[pos + d], s1v = p.rope_sin[pos + d + half];
            const float y0 = __fadd_rn(__fmul_rn(v0, c0v), __fmul_rn(-v1, s0v));
            const float y1 = __fadd_rn(__fmul_rn(v1, c1v), __fmul_rn(v0, s1v));
            v0 = y0; v1 = y1;
        }
        v0 = act_fn(v0, p.act); v1 = act_fn(v1, p.act);
        if (p.res) { v0 += p.res[(int64_t)m * p.ldres + c_r0]; if (has1) v1 += p.res[(int64_t)m * p.ldres + c_r1]; }
        p.y[(int64_t)m * p.ldy + c_r0] = v0;
        if (has1) p.y[(int64_t)m * p.ldy + c_r1] = v1;
        if (p.y2) {
            const int64_t base = (int64_t)m * p.ldy2 + (p.y2_step_d ? (int64_t)(*p.y2_step_d) * p.y2_step : 0);
            if (c_r0 >= p.y2_col0) p.y2[base + (c_r0 - p.y2_col0)] = v0;
            if (has1 && c_r1 >= p.y2_col0) p.y2[base + (c_r1 - p.y2_col0)] = v1;
        }
    }
}

// Few row pairs and a long K (the attention-output and MLP-down projections of a decode step): a warp walking the
// whole of K would issue its loads in several dependent rounds while most SMs idle. Here the eight warps of a CTA
// share ONE row pair, warp w taking chunks w, w + 8, w + 16, ... of K (at most four, all in flight at once), each
// lane reads its slice of the input rows straight from global memory, and the eight partial sums meet in shared
// memory. No fused norm on this path (the projections that use it take an un-normalised input).
template <int MT, bool W16>
__global__ void __launch_bounds__(256) k_gemv_ksplit(GemvW p) {
    __shared__ float part[8][MT][2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = blockIdx.x;
    pdl_launch_dependents();
    int r0, r1;
    gw_rows(p, g, r0, r1);
    GwTile<W16> t0, t1;
    gw_load<W16>(p, r0, warp, lane, t0, 8);
    gw_load<W16>(p, min(r1, p.N - 1), warp, lane, t1, 8);
    gw_prefetch_next(p);
    pdl_wait();
    float acc0[MT], acc1[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) { acc0[m] = 0.f; acc1[m] = 0.f; }
#pragma unroll
    for (int u = 0; u < GW_U; u++) {
        const int k = (warp + 8 * u) * 256 + lane * 8;
        if (k < p.K) {
            float w0[8], w1[8];
            gw_w8<W16>(t0, u, w0);
            gw_w8<W16>(t1, u, w1);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                if (m < p.M) {
                    const float4 xa = *(const float4 *)(p.x + (int64_t)m * p.ldx + k), xb = *(const float4 *)(p.x + (int64_t)m * p.ldx + k + 4);
                    const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                    for (int j = 0; j < 8; j++) { acc0[m] = fmaf(xv[j], w0[j], acc0[m]); acc1[m] = fmaf(xv[j], w1[j], acc1[m]); }
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc0[m] += __shfl_xor_sync(0xffffffffu, acc0[m], o);
            acc1[m] += __shfl_xor_sync(0xffffffffu, acc1[m], o);
        }
        if (lane == 0) { part[warp][m][0] = acc0[m]; part[warp][m][1] = acc1[m]; }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) { a0 += part[w][m][0]; a1 += part[w][m][1]; }
            acc0[m] = a0; acc1[m] = a1;
        }
        gw_epilogue<MT>(p, g, r0, r1, acc0, acc1);
    }
}

template <int MT, bool W16>
__global__ void __launch_bounds__(512) k_gemv_warp(GemvW p) {
    extern __shared__ __align__(16) float gw_xs[];          // [MT][K] input rows (normalised), then 64 floats of reduction scratch
    float *red = gw_xs + (size_t)MT * p.K;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    pdl_launch_dependents();
    const int nch = (p.K + 255) >> 8;
    int g = blockIdx.x * nwarp + warp;
    const int gstride = gridDim.x * nwarp;
    GwTile<W16> t0, t1;
    int r0 = 0, r1 = 0;
    if (g < p.ngroups) {
        gw_rows(p, g, r0, r1);
        gw_load<W16>(p, r0, 0, lane, t0);
        gw_load<W16>(p, min(r1, p.N - 1), 0, lane, t1);
    }
    gw_prefetch_next(p);
    pdl_wait();
    // ---- stage (and normalise) the input rows ----
    for (int i = tid * 4; i < MT * p.K; i += blockDim.x * 4) {
        const int m = i / p.K, k = i - m * p.K;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < p.M) v = *(const float4 *)(p.x + (int64_t)m * p.ldx + k);
        *(float4 *)(gw_xs + i) = v;
    }
    __syncthreads();
    if (p.ln_kind) {
        // Row statistics in two passes (mean, then squared deviations), as the stand-alone norm kernels take them.
        // Every warp forms them for itself from the staged row -- a few dozen elements per lane and two shuffle
        // reductions, the same value in every warp -- so no block-wide reduction is needed; the threads then
        // normalise the row in place, each its own part.
        for (int m = 0; m < MT; m++) {
            const float *xr = gw_xs + (size_t)m * p.K;
            float mean = 0.f;
            if (p.ln_kind == 1) {
                float part = 0.f;
                for (int k = lane * 4; k < p.K; k += 128) { const float4 v = *(const float4 *)(xr + k); part += (v.x + v.y) + (v.z + v.w); }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                mean = part / (float)p.K;
            }
            float part = 0.f;
            for (int k = lane * 4; k < p.K; k += 128) {
                const float4 v = *(const float4 *)(xr + k);
                const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
                part += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            const float rs = 1.0f / sqrtf(part / (float)p.K + p.ln_eps);
            __syncthreads();                                  // every warp has read the raw row
            for (int k = tid * 4; k < p.K; k += blockDim.x * 4) {
                float4 v = *(float4 *)(gw_xs + (size_t)m * p.K + k);
                float4 lw = make_float4(1.f, 1.f, 1.f, 1.f), lb = make_float4(0.f, 0.f, 0.f, 0.f);
                if (p.ln_w) lw = __ldg((const float4 *)(p.ln_w + k));
                if (p.ln_b) lb = __ldg((const float4 *)(p.ln_b + k));
                v.x = __fadd_rn(__fmul_rn(__fmul_rn(v.x - mean, rs), lw.x), lb.x);
                v.y = __fadd_rn(__fmul_rn(__fmul_rn(v.y - mean, rs), lw.y), lb.y);
                v.z = __fadd_rn(__fmul_rn(__fmul_rn(v.z - mean, rs), lw.z), lb.z);
                v.w = __fadd_rn(__fmul_rn(__fmul_rn(v.w - mean, rs), lw.w), lb.w);
                *(float4 *)(gw_xs + (size_t)m * p.K + k) = v;
            }
        }
        __syncthreads();
    }
    // ---- row pairs ----
    for (; g < p.ngroups; g += gstride) {
        float acc0[MT], acc1[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) { acc0[m] = 0.f; acc1[m] = 0.f; }
        const int64_t rr1 = min(r1, p.N - 1);
        for (int c0 = 0; c0 < nch; c0 += GW_U) {
            if (c0 > 0) { gw_load<W16>(p, r0, c0, lane, t0); gw_load<W16>(p, rr1, c0, lane, t1); }
#pragma unroll
            for (int u = 0; u < GW_U; u++) {
                const int k = (c0 + u) * 256 + lane * 8;
                if (k < p.K) {
                    float w0[8], w1[8];
                    gw_w8<W16>(t0, u, w0);
                    gw_w8<W16>(t1, u, w1);
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        const float4 xa = *(const float4 *)(gw_xs + (size_t)m * p.K + k), xb = *(const float4 *)(gw_xs + (size_t)m * p.K + k + 4);
                        const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                        for (int j = 0; j < 8; j++) { acc0[m] = fmaf(xv[j], w0[j], acc0[m]); acc1[m] = fmaf(xv[j], w1[j], acc1[m]); }
                    }
                }
            }
        }
        // the next pair's first loads go out before this pair's reduction and epilogue
        const int gn = g + gstride;
        int n0 = r0, n1 = r1;
        const int c_r0 = r0, c_r1 = r1;
        if (gn < p.ngroups) {
            gw_rows(p, gn, n0, n1);
            gw_load<W16>(p, n0, 0, lane, t0);
            gw_load<W16>(p, min(n1, p.N - 1), 0, lane, t1);
        }
        r0 = n0; r1 = n1;
#pragma unroll
        for (int m = 0; m < MT; m++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                acc0[m] += __shfl_xor_sync(0xffffffffu, acc0[m], o);
                acc1[m] += __shfl_xor_sync(0xffffffffu, acc1[m], o);
            }
        }
        if (lane == 0) gw_epilogue<MT>(p, g, c_r0, c_r1, acc0, acc1);
    }
}

bool gemv_warp_takes(const GemmArgs &g) {
    static const bool off = getenv("NCM_B200_OLD_GEMV") != nullptr;
    if (off || !gemv_fusable(g)) return false;
    if (g.M > 4 || (g.K % 8) != 0 || g.K < 64) return false;
    if (g.res && g.res == g.y && g.gv_pair_half) return false;
    if (g.W16 && (((uintptr_t)g.W16 & 15) != 0)) return false;
    const size_t smem = (size_t)(g.M <= 1 ? 1 : g.M <= 2 ? 2 : 4) * g.K * 4 + 256;
    return smem <= 200 * 1024;
}

template <int MT, bool W16>
static void launch_gemv_warp(const GemvW &p, int threads, int grid, size_t smem) {
    static size_t set = 0;
    if (smem > set) {
        CUDA_CHECK(cudaFuncSetAttribute((k_gemv_warp<MT, W16>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024)));
        set = 200 * 1024;
    }
    LAUNCH_PDL((k_gemv_warp<MT, W16>), grid, threads, smem, p);
}

static void gemv_warp(const GemmArgs &g) {
    GemvW p;
    p.x = g.x; p.ldx = g.ldx ? g.ldx : g.K; p.W = g.W; p.W16 = g.W16; p.bias = g.bias;
    p.res = g.res; p.ldres = g.ldres ? g.ldres : g.N;
    p.y = g.y; p.ldy = g.ldy ? g.ldy : (g.gv_pair_half ? g.gv_pair_half : g.N);
    p.M = (int)g.M; p.N = g.N; p.K = g.K; p.act = g.act;
    p.ln_kind = g.ln_kind; p.ln_w = g.ln_w; p.ln_b = g.ln_b; p.ln_eps = g.ln_eps;
    p.y2 = g.y2; p.y2_col0 = g.y2_col0; p.ldy2 = g.ldy2; p.y2_step_d = g.y2_step_d; p.y2_step = g.y2_step;
    p.pair_half = g.gv_pair_half;
    p.rope_cos = g.gv_rope_cos; p.rope_sin = g.gv_rope_sin; p.rope_pos = g.gv_rope_pos; p.rope_step_d = g.gv_rope_step_d;
    p.rope_pos_step = g.gv_rope_pos_step; p.rope_cols = g.gv_rope_cos ? g.gv_rope_cols : 0; p.hd = g.gv_hd > 0 ? g.gv_hd : 2;
    if (p.pair_half && g.N != 2 * p.pair_half) fatal("gemv: gated pairs need N = 2 * half");
    if (p.rope_cos && ((p.rope_cols % p.hd) || (p.hd & 1) || ((g.N - p.rope_cols) & 1))) fatal("gemv: rotary heads do not tile the columns");
    p.ngroups = p.pair_half ? p.pair_half : (g.N + 1) / 2;
    static const bool pf_ok = !getenv("NCM_B200_NO_GEMV_PREFETCH");
    p.pf = (pf_ok && g.pf_next && ((uintptr_t)g.pf_next & 15) == 0) ? (const char *)g.pf_next : nullptr;
    p.pf_bytes = g.pf_next_bytes;
    const int mt = g.M <= 1 ? 1 : g.M <= 2 ? 2 : 4;
    const size_t smem = (size_t)mt * g.K * 4 + 256;
    // warps per CTA: as many as still leave every SM a CTA; CTAs: one or two per SM, persistent over the pairs
    const int sms = ctx().sm_count;
    static const int thr_env = getenv("NCM_B200_GW_THREADS") ? atoi(getenv("NCM_B200_GW_THREADS")) : 0;     // A/B knobs
    static const int psm_env = getenv("NCM_B200_GW_PER_SM") ? atoi(getenv("NCM_B200_GW_PER_SM")) : 0;
    int threads = 512;
    while (threads > 128 && (p.ngroups + (threads / 32) - 1) / (threads / 32) < sms) threads >>= 1;
    if (thr_env >= 32 && thr_env <= 512) threads = thr_env;
    const int per_sm = psm_env > 0 ? psm_env : (smem > 100 * 1024 ? 1 : 2);
    int grid = (p.ngroups + (threads / 32) - 1) / (threads / 32);
    if (grid > sms * per_sm) grid = sms * per_sm;
    if (grid < 1) grid = 1;
    const bool w16 = g.W16 != nullptr;
    // few pairs, long K, no fused norm: the eight warps of a CTA share one pair (see k_gemv_ksplit)
    static const bool ksplit_ok = !getenv("NCM_B200_NO_GEMV_KSPLIT");
    const int nch = (g.K + 255) / 256;
    if (ksplit_ok && !g.ln_kind && nch > GW_U && nch <= 8 * GW_U && p.ngroups <= sms * 8) {
        if (mt == 1) { if (w16) LAUNCH_PDL((k_gemv_ksplit<1, true>), p.ngroups, 256, 0, p); else LAUNCH_PDL((k_gemv_ksplit<1, false>), p.ngroups, 256, 0, p); }
        else if (mt == 2) { if (w16) LAUNCH_PDL((k_gemv_ksplit<2, true>), p.ngroups, 256, 0, p); else LAUNCH_PDL((k_gemv_ksplit<2, false>), p.ngroups, 256, 0, p); }
        else { if (w16) LAUNCH_PDL((k_gemv_ksplit<4, true>), p.ngroups, 256, 0, p); else LAUNCH_PDL((k_gemv_ksplit<4, false>), p.ngroups, 256, 0, p); }
        return;
    }
    if (mt == 1) { if (w16) launch_gemv_warp<1, true>(p, threads, grid, smem); else launch_gemv_warp<1, false>(p, threads, grid, smem); }
    else if (mt == 2) { if (w16) launch_gemv_warp<2, true>(p, threads, grid, smem); else launch_gemv_warp<2, false>(p, threads, grid, smem); }
    else { if (w16) launch_gemv_warp<4, true>(p, threads, grid, smem); else launch_gemv_warp<4, false>(p, threads, grid, smem); }
}

void gemm_simt(const GemmArgs &g) {
    if (g.M <= 0 || g.N <= 0) return;
    if (g.glu) fatal("gemm_simt: fused gated epilogue is a tensor-core engine feature");
    if (gemv_warp_takes(g)) {
        ProfScope ps(NCMB_K_GEMM, 2.0 * (double)g.M * g.N * g.K, (g.W16 ? 2.0 : 4.0) * (double)g.N * g.K);
        gemv_warp(g);
        return;
    }
    if (g.gv_pair_half || g.gv_rope_cos) fatal("gemm_simt: gated-pair / rotary epilogue on a call the warp GEMV does not take");
    GemmDev d;
    d.x = g.x; d.ldx = g.ldx ? g.ldx : g.K;
    d.W = g.W; d.bias = g.bias;
    d.res = g.res; d.ldres = g.ldres ? g.ldres : g.N;
    d.y = g.y; d.ldy = g.ldy ? g.ldy : g.N;
    d.M = g.M; d.N = g.N; d.K = g.K; d.act = g.act;
    d.vec = (g.K % 4 == 0) && (d.ldx % 4 == 0) && (((uintptr_t)g.x & 15) == 0) && (((uintptr_t)g.W & 15) == 0);
    d.W16 = (g.M <= 16 && d.vec) ? g.W16 : nullptr;
    d.ln_kind = g.ln_kind; d.ln_w = g.ln_w; d.ln_b = g.ln_b; d.ln_eps = g.ln_eps;
    d.y2 = g.y2; d.y2_col0 = g.y2_col0; d.ldy2 = g.ldy2; d.y2_step_d = g.y2_step_d; d.y2_step = g.y2_step;
    if ((g.ln_kind || g.y2) && !(g.M <= 16 && d.vec)) fatal("gemm_simt: fused norm / second output on a call the GEMV kernel does not take");
    ProfScope ps(NCMB_K_GEMM, 2.0 * (double)g.M * g.N * g.K,
                 4.0 * ((double)g.M * g.K + (double)g.N * g.K + (double)g.M * g.N));
    // Few rows: the weights dominate the traffic and a 64x64 / 128x128 tiling would leave most
    // SMs idle, so stream each weight row once through one warp (decode-time GEMV / skinny GEMM).
    if (g.M <= 16 && d.vec) {
        // columns per CTA: more of them when there are many, so a CTA moves tens of KB per launch-and-reduce
        // cycle and a few waves cover the matrix (N = vocabulary: 16 columns; MLP widths: 8)
        const int nc = (g.M <= 2 && g.N >= 32768) ? 16 : (g.M <= 4 && g.N >= 2048) ? 8 : 4;
        unsigned grid = (unsigned)cdiv(g.N, nc);
        if (nc == 16) {
            if (g.M <= 1) LAUNCH_PDL((k_gemv<1, 16, 1>), grid, 256, 0, d);
            else LAUNCH_PDL((k_gemv<2, 16, 1>), grid, 256, 0, d);
        } else if (nc == 8) {
            if (g.M <= 1) LAUNCH_PDL((k_gemv<1, 8, 2>), grid, 256, 0, d);
            else if (g.M <= 2) LAUNCH_PDL((k_gemv<2, 8, 1>), grid, 256, 0, d);
            else LAUNCH_PDL((k_gemv<4, 8, 1>), grid, 256, 0, d);
        } else {
            if (g.M <= 1) LAUNCH_PDL((k_gemv<1, 4, 3>), grid, 256, 0, d);
            else if (g.M <= 2) LAUNCH_PDL((k_gemv<2, 4, 3>), grid, 256, 0, d);
            else if (g.M <= 4) LAUNCH_PDL((k_gemv<4, 4, 3>), grid, 256, 0, d);
            else LAUNCH_PDL((k_gemv<8, 4, 2>), grid, 256, 0, d);
        }
        return;
    }
    if (g.M <= 16) {
        unsigned grid = grid1d((int64_t)g.N * 32, 256);
        if (g.M <= 1) LAUNCH(k_gemm_skinny<1>, grid, 256, 0, d);
        else if (g.M <= 4) LAUNCH(k_gemm_skinny<4>, grid, 256, 0, d);
        else LAUNCH(k_gemm_skinny<8>, grid, 256, 0, d);
        return;
    }
    int64_t big = cdiv(g.M, 128) * cdiv(g.N, 128);
    if (big >= ctx().sm_count) {
        dim3 grid((unsigned)cdiv(g.N, 128), (unsigned)cdiv(g.M, 128));
        LAUNCH((k_gemm_tiled<128, 128, 16>), grid, 256, 0, d);
    } else {
        dim3 grid((unsigned)cdiv(g.N, 64), (unsigned)cdiv(g.M, 64));
        LAUNCH((k_gemm_tiled<64, 64, 16>), grid, 64, 0, d);
    }
}

bool gemv_fusable(const GemmArgs &g) {
    int64_t ldx = g.ldx ? g.ldx : g.K;
    return g.M <= 16 && g.M > 0 && !g.glu && !g.x_lo && !g.y_lo && (g.K % 4 == 0) && (ldx % 4 == 0) &&
           (((uintptr_t)g.x & 15) == 0) && (((uintptr_t)g.W & 15) == 0) &&
           (!g.ln_w || ((uintptr_t)g.ln_w & 15) == 0) && (!g.ln_b || ((uintptr_t)g.ln_b & 15) == 0);
}

void gemm(const GemmArgs &a) {
    const int mode = ctx().gemm_mode;
    // a pre-split input names its engine; otherwise mode 3 prefers the fp16-pair kernel
    if (a.x_lo && a.x_fmt == SPLIT_H16) {
        if (!gemm_h3_supported(a)) fatal("gemm: fp16-pair operands for a shape the fp16-pair kernel does not take (M=%lld N=%d K=%d)", (long long)a.M, a.N, a.K);
        gemm_h3(a); return;
    }
    if (mode >= 3 && !a.x_lo && gemm_h3_supported(a)) { gemm_h3(a); return; }
    if (mode >= 1 && gemm_tc_supported(a)) { gemm_tc(a); return; }
    if (a.x_lo || a.y_lo) fatal("gemm: split operands reached the CUDA-core engine (M=%lld N=%d K=%d)", (long long)a.M, a.N, a.K);
    gemm_simt(a);
}

} // namespace ncmb

extern "C" void linear_fwd(const float *x, const float *W, const float *b, float *y, int64_t batch, int M, int K) {
    ncmb::ensure_device();
    ncmb::GemmArgs a;
    a.x = x; a.ldx = K; a.W = W; a.bias = b; a.y = y; a.ldy = M;
    a.M = batch; a.N = M; a.K = K;
    ncmb::gemm(a);
}
